// Varlen causal prefill attention, tcgen05 / TMEM, persistent, ping-ponged halves with
// double-buffered S: the fast path.  Replaces flash_attn_varlen_func as called at
// nanovllm/layers/attention.py:64-70, for dense K/V and for K/V read from the paged cache.
//
// Same skeleton as prefill_attn_tc2.cu (one persistent CTA per SM; an item = 2 * QT query tokens of
// one kv head = two 128-row halves A and B sharing every K/V tile; TMA producer warp, one MMA-issuing
// thread, one softmax warpgroup per half, tickets from an atomic counter), with the K/V step cut to
// 64 keys so that each half owns TWO S buffers in TMEM:
//   TMEM columns   A: S0 [0,64) S1 [64,128)   B: S0 [128,192) S1 [192,256)   O_A [256,384)  O_B [384,512)
// P(j) (bf16) overwrites the first 32 columns of the S buffer it was computed from.  The issuer runs
// S_X(j+2) right after PV_X(j), so S_X(j+1) is already in TMEM when the softmax finishes tile j: the
// softmax never waits for the tensor core, and it loads S(j+1) into registers before it starts the
// arithmetic of tile j (64 + 64 registers), which hides the TMEM load latency as well.
#include <atomic>
#include <type_traits>

#include "../../include/b200_attn.h"
#include "kernels.cuh"
#include "tcgen05.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kT3Kv = 64;                    // keys per step
constexpr int kT3QSub = 128 * 128;           // Q: one 64-column sub-tile of a 128-row tile (bytes)
constexpr int kT3QTile = 2 * kT3QSub;        // 32 KiB
constexpr int kT3KvSub = kT3Kv * 128;        // K/V: one 64-column sub-tile of a 64-row tile (8 KiB)
constexpr int kT3KvTile = 2 * kT3KvSub;      // 16 KiB
constexpr int kT3Threads = 384;              // warpgroup 0: producer, issuer, two idle warps; 1, 2: softmax A, B
constexpr int kT3Ring = 4;                   // K ring depth and V ring depth
constexpr int kT3Items = 4;
constexpr int kT3MaxSeqSmem = 1024;
constexpr float kT3Rescale = 8.0f;

static __device__ int g_status_prefill_tc3 = 0;
static __device__ unsigned int g_prefill_ticket3 = 0;
#ifdef B200_TRACE
__device__ unsigned long long g_pf3_trace[8 * 8];
#define CK3(var) do { const long long now_ = clock64(); var += now_ - ck_t0; ck_t0 = now_; } while (0)
#else
#define CK3(var) do { } while (0)
#endif

struct T3Item {
  int seq;        // -1: no more work
  int h;
  int q_row;      // global row of the block's first query token
  int tq0;        // that token's index within the sequence
  int Lq, Lk;
  int k_begin;    // dense K/V: first row of the sequence
  int n[2];       // 64-key steps each half needs (n[1] == 0: half B is empty or sees nothing)
};

__global__ void __launch_bounds__(kT3Threads, 1)
prefill_attn_tc3_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;                              // [2][32 KiB]
  unsigned char* sK = smem + 2 * kT3QTile;               // [kT3Ring][16 KiB]
  unsigned char* sV = sK + kT3Ring * kT3KvTile;          // [kT3Ring][16 KiB]
  int* s_slot = reinterpret_cast<int*>(sV + kT3Ring * kT3KvTile);
  __shared__ __align__(8) uint64_t bar_item_full[kT3Items], bar_item_empty[kT3Items];
  __shared__ __align__(8) uint64_t bar_q_full[2], bar_q_empty[2];
  __shared__ __align__(8) uint64_t bar_k_full[kT3Ring], bar_k_empty[kT3Ring], bar_v_full[kT3Ring], bar_v_empty[kT3Ring];
  __shared__ __align__(8) uint64_t bar_s_full[2][2], bar_p_full[2][2], bar_pv_done[2][2], bar_o_final[2], bar_o_free[2];
  __shared__ __align__(16) T3Item s_item[kT3Items];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, QT = p.QT, QB = 2 * p.QT;
  const bool slot_in_smem = p.batch <= kT3MaxSeqSmem;

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < kT3Items; ++i) { mbar_init(&bar_item_full[i], 1); mbar_init(&bar_item_empty[i], 9); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_q_full[i], 1);
      mbar_init(&bar_q_empty[i], 1);
      mbar_init(&bar_o_final[i], 1);
      mbar_init(&bar_o_free[i], 4);
      for (int b = 0; b < 2; ++b) {
        mbar_init(&bar_s_full[i][b], 1);
        mbar_init(&bar_p_full[i][b], 4);
        mbar_init(&bar_pv_done[i][b], 1);
      }
    }
    for (int i = 0; i < kT3Ring; ++i) {
      mbar_init(&bar_k_full[i], 1);
      mbar_init(&bar_k_empty[i], 1);
      mbar_init(&bar_v_full[i], 1);
      mbar_init(&bar_v_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (slot_in_smem)
    for (int i = tid; i <= p.batch; i += kT3Threads) s_slot[i] = __ldg(p.cu_q + i) / QB + i;
  if (warp == 1) {
    tc::tmem_alloc(&s_tmem_base, 512);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;" ::: "memory");
    if (warp == 0) {
      // ================================ TMA producer ================================
      if (lane == 0) {
        tma_prefetch_desc(&map_q);
        tma_prefetch_desc(&map_k);
        tma_prefetch_desc(&map_v);
        const unsigned int n_items = static_cast<unsigned int>(p.n_slots) * p.Hkv;
        int n_pub = 0;
        int kt = 0, vt = 0;
        bool ok = true;
        while (ok) {
          const unsigned int tk = atomicAdd(&g_prefill_ticket3, 1u);
          if (tk == n_items + gridDim.x - 1) atomicExch(&g_prefill_ticket3, 0u);
          T3Item it;
          it.seq = -1;
          if (tk < n_items) {
            const int h = tk % p.Hkv;
            const int x = p.n_slots - 1 - static_cast<int>(tk / p.Hkv);   // later (heavier) blocks first
            int lo = 0, hi = p.batch;
            while (hi - lo > 1) {
              const int mid = (lo + hi) >> 1;
              const int f = slot_in_smem ? s_slot[mid] : __ldg(p.cu_q + mid) / QB + mid;
              if (f <= x) lo = mid; else hi = mid;
            }
            const int q_begin = __ldg(p.cu_q + lo), q_end = __ldg(p.cu_q + lo + 1);
            const int Lq = q_end - q_begin;
            const int qb = x - (q_begin / QB + lo);
            if (qb < 0 || qb * QB >= Lq) continue;                        // slot owns no query block
            const int k_begin = __ldg(p.cu_k + lo);
            const int Lk = __ldg(p.cu_k + lo + 1) - k_begin;
            const int shift = Lk - Lq;
            const int tq0 = qb * QB;
            const int endA = min(tq0 + QT, Lq), endB = min(tq0 + QB, Lq);
            it.seq = lo;
            it.h = h;
            it.q_row = q_begin + tq0;
            it.tq0 = tq0;
            it.Lq = Lq;
            it.Lk = Lk;
            it.k_begin = k_begin;
            it.n[0] = max(0, (min(Lk, shift + endA) + kT3Kv - 1) / kT3Kv);
            it.n[1] = tq0 + QT < Lq ? max(0, (min(Lk, shift + endB) + kT3Kv - 1) / kT3Kv) : 0;
          }
          const int is = n_pub % kT3Items;
          if (!mbar_wait(&bar_item_empty[is], ((n_pub / kT3Items) & 1) ^ 1, abort_flag)) { ok = false; break; }
          s_item[is] = it;
          mbar_arrive(&bar_item_full[is]);
          if (it.seq < 0) break;
          const uint32_t qph = (n_pub & 1) ^ 1;
          for (int hx = 0; hx < 2; ++hx) {
            if (!mbar_wait(&bar_q_empty[hx], qph, abort_flag)) { ok = false; break; }
            if (hx == 1 && it.tq0 + QT >= it.Lq) { mbar_arrive(&bar_q_full[1]); continue; }
            mbar_expect_tx(&bar_q_full[hx], kT3QTile);
            tma_load_3d(sQ + hx * kT3QTile, &map_q, &bar_q_full[hx], 0, it.h * G, it.q_row + hx * QT);
            tma_load_3d(sQ + hx * kT3QTile + kT3QSub, &map_q, &bar_q_full[hx], 64, it.h * G, it.q_row + hx * QT);
          }
          if (!ok) break;
          ++n_pub;
          const int n = max(it.n[0], it.n[1]);
          const int* bt_row = p.block_tables ? p.block_tables + it.seq * p.bt_row_stride : nullptr;
          for (int j = 0; j < n; ++j) {
            int row0;
            if (bt_row) {
              const int tok0 = j * kT3Kv;
              const int col = tok0 / p.block_size;
              const long long blk = col < p.bt_cols ? bt_row[col] : -1;
              row0 = (blk >= 0 && blk < p.num_blocks) ? static_cast<int>(blk * p.block_size + (tok0 - col * p.block_size))
                                                      : -kT3Kv;
            } else {
              row0 = it.k_begin + j * kT3Kv;
            }
            const int ks = kt % kT3Ring;
            if (!mbar_wait(&bar_k_empty[ks], ((kt / kT3Ring) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&bar_k_full[ks], kT3KvTile);
            tma_load_3d(sK + ks * kT3KvTile, &map_k, &bar_k_full[ks], 0, it.h, row0);
            tma_load_3d(sK + ks * kT3KvTile + kT3KvSub, &map_k, &bar_k_full[ks], 64, it.h, row0);
            ++kt;
            const int vs = vt % kT3Ring;
            if (!mbar_wait(&bar_v_empty[vs], ((vt / kT3Ring) & 1) ^ 1, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&bar_v_full[vs], kT3KvTile);
            tma_load_3d(sV + vs * kT3KvTile, &map_v, &bar_v_full[vs], 0, it.h, row0);
            tma_load_3d(sV + vs * kT3KvTile + kT3KvSub, &map_v, &bar_v_full[vs], 64, it.h, row0);
            ++vt;
          }
        }
      }
    } else if (warp == 1) {
      // ================================ MMA issuer ================================
      if (lane == 0) {
        constexpr uint32_t idesc_qk = tc::idesc_bf16_f32(128, 64, false, false);
        constexpr uint32_t idesc_pv = tc::idesc_bf16_f32(128, 128, false, true);
        const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
        int n_item = 0;
        int kbase = 0, vbase = 0;     // ring position of the item's tile 0
        int cnt[2] = {0, 0};          // 64-key tiles of each half so far (S buffer = cnt & 1, phase = (cnt >> 1) & 1)
        int no[2] = {0, 0};           // items whose O was handed to the epilogue, per half
        bool ok = true;
        // S_X(t) = Q_X K_t^T into the half's buffer (cnt_item_base + t) & 1
        auto issue_s = [&](int hx, int buf, int kslot) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t qoff = (ks >> 2) * kT3QSub + (ks & 3) * 32;
            const uint32_t koff = (ks >> 2) * kT3KvSub + (ks & 3) * 32;
            tc::mma_ss(tmem + hx * 128 + buf * 64, tc::smem_desc_sw128(q_addr + hx * kT3QTile + qoff, 16, 1024),
                       tc::smem_desc_sw128(k_addr + kslot * kT3KvTile + koff, 16, 1024), idesc_qk, ks > 0);
          }
          tc::commit(&bar_s_full[hx][buf]);
        };
        auto issue_pv = [&](int hx, int buf, int vslot, bool accumulate) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            tc::mma_ts(tmem + 256 + hx * 128, tmem + hx * 128 + buf * 64 + ks * 8,
                       tc::smem_desc_sw128(v_addr + vslot * kT3KvTile + ks * 2048, kT3KvSub, 1024), idesc_pv,
                       accumulate || ks > 0);
          tc::commit(&bar_pv_done[hx][buf]);
        };
        while (ok) {
          const int is = n_item % kT3Items;
          if (!mbar_wait(&bar_item_full[is], (n_item / kT3Items) & 1, abort_flag)) break;
          const T3Item it = s_item[is];
          mbar_arrive(&bar_item_empty[is]);
          if (it.seq < 0) break;
          const int nn[2] = {it.n[0], it.n[1]};
          const int n = max(nn[0], nn[1]);
          const uint32_t qph = n_item & 1;
          if (!mbar_wait(&bar_q_full[0], qph, abort_flag) || !mbar_wait(&bar_q_full[1], qph, abort_flag)) break;
          // S for K tile t, both halves, then release the K slot (and the Q tiles after their last use)
          auto s_step = [&](int t) -> bool {
            const int kslot = (kbase + t) % kT3Ring;
            if (!mbar_wait(&bar_k_full[kslot], ((kbase + t) / kT3Ring) & 1, abort_flag)) return false;
            tc::fence_after_sync();
            for (int hx = 0; hx < 2; ++hx) {
              if (t >= nn[hx]) continue;
              issue_s(hx, (cnt[hx] + t) & 1, kslot);
              if (t == nn[hx] - 1) tc::commit(&bar_q_empty[hx]);
            }
            tc::commit(&bar_k_empty[kslot]);
            return true;
          };
          for (int hx = 0; hx < 2; ++hx)
            if (nn[hx] == 0) tc::commit(&bar_q_empty[hx]);
          for (int t = 0; t < 2 && t < n && ok; ++t) ok = s_step(t);
          for (int j = 0; j < n && ok; ++j) {
            const int vslot = (vbase + j) % kT3Ring;
            const uint32_t vph = ((vbase + j) / kT3Ring) & 1;
            for (int hx = 0; hx < 2 && ok; ++hx) {
              if (j >= nn[hx]) continue;
              const int c = cnt[hx] + j, buf = c & 1;
              if (!mbar_wait(&bar_p_full[hx][buf], (c >> 1) & 1, abort_flag)) { ok = false; break; }
              if (j == 0 && !mbar_wait(&bar_o_free[hx], (no[hx] & 1) ^ 1, abort_flag)) { ok = false; break; }
              if (!mbar_wait(&bar_v_full[vslot], vph, abort_flag)) { ok = false; break; }
              tc::fence_after_sync();
              issue_pv(hx, buf, vslot, j > 0);
              if (j == nn[hx] - 1) { tc::commit(&bar_o_final[hx]); ++no[hx]; }
            }
            if (!ok) break;
            tc::commit(&bar_v_empty[vslot]);
            if (j + 2 < n) ok = s_step(j + 2);   // the S buffers of tile j are free: their PV is in the queue ahead
          }
          cnt[0] += nn[0];
          cnt[1] += nn[1];
          kbase += n;
          vbase += n;
          ++n_item;
        }
      }
    }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;" ::: "memory");
    // ================================ softmax / epilogue ================================
    const int hx = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tmem_s = tmem + hx * 128, tmem_o = tmem + 256 + hx * 128;
    const float c = p.scale_log2;
    int n_item = 0, n_final = 0, vt_base = 0;
    int cnt = 0;        // 64-key tiles of this half so far
    bool ok = true;
#ifdef B200_TRACE
    long long ck_wait = 0, ck_max = 0, ck_exp = 0, ck_sig = 0, ck_epi = 0, ck_first = 0, ck_tiles = 0, ck_t0 = 0;
#endif
    while (ok) {
      const int is = n_item % kT3Items;
      if (!mbar_wait(&bar_item_full[is], (n_item / kT3Items) & 1, abort_flag)) break;
      const T3Item it = s_item[is];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_item_empty[is]);
      if (it.seq < 0) break;
      ++n_item;
      const int nx = it.n[hx];
      const int n_all = max(it.n[0], it.n[1]);
      const int shift = it.Lk - it.Lq;
      const int tok = it.tq0 + hx * QT + r / G;
      const bool row_ok = r < QT * G && tok < it.Lq;
      const int kmax = row_ok ? shift + tok : -1;
      const int first_row_kmax = shift + it.tq0 + hx * QT;
      float m_used = -INFINITY, l = 0.f;
      // Two register images of an S tile: even tiles of the item live in sa, odd tiles in sb; while one
      // is being turned into P the other is being loaded.
      uint32_t sv[2][2][32];
#ifdef B200_TRACE
      ck_t0 = clock64();
#endif
      if (nx > 0) {
        if (!mbar_wait(&bar_s_full[hx][cnt & 1], (cnt >> 1) & 1, abort_flag)) break;
        tc::fence_after_sync();
        tc::ld_32x32b_x32(tmem_s + lane_base + (cnt & 1) * 64, sv[0][0]);
        tc::ld_32x32b_x32(tmem_s + lane_base + (cnt & 1) * 64 + 32, sv[0][1]);
        tc::wait_ld();
      }
      CK3(ck_first);
      // PAR is the parity of the tile within the item: a literal, so that every register index below is static
      auto step = [&](int j, auto par_tag) -> bool {
        constexpr int PAR = decltype(par_tag)::value;
        uint32_t (&cur)[2][32] = sv[PAR];
        uint32_t (&nxt)[2][32] = sv[PAR ^ 1];
        const int cj = cnt + j, buf = cj & 1;
        // S of the next tile is already in TMEM (or will be in a moment): start loading it now
        if (j + 1 < nx) {
          if (!mbar_wait(&bar_s_full[hx][buf ^ 1], ((cj + 1) >> 1) & 1, abort_flag)) return false;
          tc::fence_after_sync();
          tc::ld_32x32b_x32(tmem_s + lane_base + (buf ^ 1) * 64, nxt[0]);
          tc::ld_32x32b_x32(tmem_s + lane_base + (buf ^ 1) * 64 + 32, nxt[1]);
        }
#ifdef B200_TRACE
        ++ck_tiles;
#endif
        CK3(ck_wait);
        const int key0 = j * kT3Kv;
        if (key0 + kT3Kv - 1 > first_row_kmax) {
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (key0 + h2 * 32 + i > kmax) cur[h2][i] = 0xff800000u;   // -inf
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        float mx4 = -INFINITY, mx5 = -INFINITY, mx6 = -INFINITY, mx7 = -INFINITY;
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            mx0 = fmaxf(mx0, __uint_as_float(cur[h2][i]));
            mx1 = fmaxf(mx1, __uint_as_float(cur[h2][i + 1]));
            mx2 = fmaxf(mx2, __uint_as_float(cur[h2][i + 2]));
            mx3 = fmaxf(mx3, __uint_as_float(cur[h2][i + 3]));
            mx4 = fmaxf(mx4, __uint_as_float(cur[h2][i + 4]));
            mx5 = fmaxf(mx5, __uint_as_float(cur[h2][i + 5]));
            mx6 = fmaxf(mx6, __uint_as_float(cur[h2][i + 6]));
            mx7 = fmaxf(mx7, __uint_as_float(cur[h2][i + 7]));
          }
        }
        const float mx = fmaxf(fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)), fmaxf(fmaxf(mx4, mx5), fmaxf(mx6, mx7)));
        const float m_new = fmaxf(m_used, mx);
        if (j == 0) {
          m_used = m_new;
        } else {
          const bool grow = (m_new - m_used) * c > kT3Rescale;
          if (__any_sync(0xffffffffu, grow)) {
            // rare: O must not be in use by the previous tile's PV while it is rescaled
            if (!mbar_wait(&bar_pv_done[hx][buf ^ 1], ((cj - 1) >> 1) & 1, abort_flag)) return false;
            tc::fence_after_sync();
            const float alpha = grow ? fast_exp2((m_used - m_new) * c) : 1.f;
            if (grow) { m_used = m_new; l *= alpha; }
            for (int cch = 0; cch < 8; ++cch) {
              uint32_t v[16];
              tc::ld_32x32b_x16(tmem_o + lane_base + cch * 16, v);
              tc::wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
              tc::st_32x32b_x16(tmem_o + lane_base + cch * 16, v);
            }
          }
        }
        CK3(ck_max);
        const float mc = (m_used == -INFINITY ? 0.f : m_used) * c;
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            const float p0 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i]), c, -mc));
            const float p1 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i + 1]), c, -mc));
            const float p2 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i + 2]), c, -mc));
            const float p3 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i + 3]), c, -mc));
            const float p4 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i + 4]), c, -mc));
            const float p5 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i + 5]), c, -mc));
            const float p6 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i + 6]), c, -mc));
            const float p7 = fast_exp2(fmaf(__uint_as_float(cur[h2][2 * i + 7]), c, -mc));
            l0 += p0 + p1;
            l1 += p2 + p3;
            l2 += p4 + p5;
            l3 += p6 + p7;
            pk[i] = pack_bf16(p0, p1);
            pk[i + 1] = pack_bf16(p2, p3);
            pk[i + 2] = pack_bf16(p4, p5);
            pk[i + 3] = pack_bf16(p6, p7);
          }
          tc::st_32x32b_x16(tmem_s + lane_base + buf * 64 + h2 * 16, pk);
        }
        l += (l0 + l1) + (l2 + l3);
        CK3(ck_exp);
        if (key0 + kT3Kv > it.Lk) {
          // ragged last tile of the sequence: V rows past its end are foreign data; zero them so
          // that 0 * garbage cannot turn into NaN inside the tensor core
          const int vt = vt_base + j;
          if (!mbar_wait(&bar_v_full[vt % kT3Ring], (vt / kT3Ring) & 1, abort_flag)) return false;
          if (r < kT3Kv && key0 + r >= it.Lk) {
            unsigned char* vrow = sV + (vt % kT3Ring) * kT3KvTile + r * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              *reinterpret_cast<uint4*>(vrow + i * 16) = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(vrow + kT3KvSub + i * 16) = make_uint4(0, 0, 0, 0);
            }
          }
          fence_proxy_async_smem();
        }
        tc::wait_ld();      // next tile's S is in registers (this overlapped the arithmetic above)
        tc::wait_st();      // P is in TMEM
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_p_full[hx][buf]);   // one arrival per warp
        CK3(ck_sig);
        return true;
      };
      for (int j = 0; j < nx && ok; j += 2) {
        ok = step(j, std::integral_constant<int, 0>{});
        if (ok && j + 1 < nx) ok = step(j + 1, std::integral_constant<int, 1>{});
      }
      if (!ok) break;
      cnt += nx;
      vt_base += n_all;
      if (nx > 0) {
        if (!mbar_wait(&bar_o_final[hx], n_final & 1, abort_flag)) break;
        ++n_final;
        tc::fence_after_sync();
        const float inv = l > 0.f ? 1.f / l : 0.f;
        uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<long long>(it.q_row + hx * QT + r / G) * p.H + it.h * G + r % G) * 128);
        // two 64-column halves of the O row at a time (registers are shared with the S images above)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t ov[2][32];
          tc::ld_32x32b_x32(tmem_o + lane_base + half * 64, ov[0]);
          tc::ld_32x32b_x32(tmem_o + lane_base + half * 64 + 32, ov[1]);
          tc::wait_ld();
          if (half == 1) {
            // O is in registers: the accumulator may be overwritten by the next item already
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_o_free[hx]);
          }
          if (row_ok) {
#pragma unroll
            for (int cch = 0; cch < 2; ++cch) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 w;
                w.x = pack_bf16(__uint_as_float(ov[cch][8 * i]) * inv, __uint_as_float(ov[cch][8 * i + 1]) * inv);
                w.y = pack_bf16(__uint_as_float(ov[cch][8 * i + 2]) * inv, __uint_as_float(ov[cch][8 * i + 3]) * inv);
                w.z = pack_bf16(__uint_as_float(ov[cch][8 * i + 4]) * inv, __uint_as_float(ov[cch][8 * i + 5]) * inv);
                w.w = pack_bf16(__uint_as_float(ov[cch][8 * i + 6]) * inv, __uint_as_float(ov[cch][8 * i + 7]) * inv);
                dst[half * 8 + cch * 4 + i] = w;
              }
            }
          }
        }
        CK3(ck_epi);
      } else if (row_ok) {
        // no visible key at all (Lk < Lq rows): zeros, as the reference's attention library does
        uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<long long>(it.q_row + hx * QT + r / G) * p.H + it.h * G + r % G) * 128);
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = make_uint4(0, 0, 0, 0);
      }
    }
#ifdef B200_TRACE
    if (hx == 0 && r == 0 && blockIdx.x < 8) {
      unsigned long long* o = g_pf3_trace + blockIdx.x * 8;
      o[0] = ck_tiles; o[1] = ck_wait; o[2] = ck_max; o[3] = ck_exp; o[4] = ck_sig; o[5] = ck_epi; o[6] = n_item; o[7] = ck_first;
    }
#endif
  }

  // ---- teardown: everyone meets, then the allocating warp frees TMEM ----
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && s_abort) atomicExch(&g_status_prefill_tc3, 1);
}

#ifdef B200_TRACE
extern "C" int b200_debug_trace_prefill3(unsigned long long* host_out, int n) {
  return static_cast<int>(cudaMemcpyFromSymbol(host_out, g_pf3_trace, sizeof(unsigned long long) * n));
}
#endif

int read_status_prefill_tc3() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_status_prefill_tc3, sizeof(int));
  return v;
}

// K/V maps must have 64-token boxes; the query-block slots are laid out for 2 * QT tokens.
int launch_prefill_tc3(PrefillParams p, const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                       cudaStream_t stream) {
  p.n_slots = p.total_q / (2 * p.QT) + p.batch;
  const size_t smem = 1024 + 2 * static_cast<size_t>(kT3QTile) + 2 * static_cast<size_t>(kT3Ring) * kT3KvTile +
                      (p.batch <= kT3MaxSeqSmem ? (p.batch + 1) * 4 : 4) + 64;
  static std::atomic<size_t> configured{0};
  if (configured.load() < smem) {
    int rc = check_cuda(cudaFuncSetAttribute(prefill_attn_tc3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "prefill_attn(tc3): cudaFuncSetAttribute");
    if (rc) return rc;
    configured.store(smem);
  }
  const int grid = sm_count();
  if (grid <= 0) return set_error(kErrNoDriver, "prefill_attn: no CUDA device");
  if (static_cast<long long>(p.n_slots) * p.Hkv > 0x7fffffffLL) return set_error(kErrBadShape, "prefill_attn: too many query blocks");
  prefill_attn_tc3_kernel<<<grid, kT3Threads, smem, stream>>>(p, map_q, map_k, map_v);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "prefill_attn(tc3) launch");
}

}  // namespace b200
