// Varlen causal prefill attention, tcgen05 / TMEM, persistent and ping-ponged: the fast path.
// Replaces flash_attn_varlen_func as called at nanovllm/layers/attention.py:64-70, for dense K/V
// and for K/V read from the paged cache.
//
// One persistent CTA per SM.  A work item is (sequence, kv head, block of 2 * QT query tokens),
// QT = 128 / G, handed out through an atomic ticket counter in reverse slot order (the last sequence first, and
// within a sequence its last, longest query block first; not sorted by work across sequences).  The two
// halves of the block ("A" = first QT tokens, "B" = next QT) are two independent 128-row tiles that
// share every K/V tile, so K/V traffic per query row is halved and, more to the point, the tensor
// core always has the other half's MMA to run while one half is in its softmax:
//   warp 0        TMA producer: draws tickets, publishes item descriptors, loads Q_A / Q_B and
//                 feeds two-deep rings of 128-token K tiles and V tiles;
//   warp 1        one elected thread issues tcgen05.mma:  S_X = Q_X K^T  (M128 N128 K16 x 8) and
//                 O_X += P_X V  (A operand = P read from TMEM, B = V as MN-major shared memory);
//   warps 4-7     softmax warpgroup of half A: thread r owns TMEM lane r = one query row; reads S
//                 with tcgen05.ld, keeps max / sum in registers, writes P (bf16) over S with
//                 tcgen05.st, rescales O in TMEM only when the row max grew by more than 2^8;
//   warps 8-11    the same for half B;
//   warps 12-15   output warpgroup: takes a finished O out of TMEM, scales it by 1 / row sum and
//                 sends it out as bf16 through TMA stores (plain stores where a box would overhang
//                 the sequence), so the softmax warpgroups never stop for output.
//   (Warps 2-3 idle; setmaxnreg: warpgroup 0 -> 80, softmax -> 184, output -> 64 registers.)
// TMEM: S_A [0,128)  S_B [128,256)  O_A [256,384)  O_B [384,512).  Every mbarrier wait is bounded.
#include "../../include/b200_attn.h"
#include "kernels.cuh"
#include "tcgen05.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kT2Kv = 128;
constexpr int kT2Sub = 128 * 128;            // one 64-column sub-tile of a 128-row tile (bytes)
constexpr int kT2Tile = 2 * kT2Sub;          // 128 rows x 128 dims bf16 = 32 KiB
constexpr int kT2Threads = 512;   // warpgroup 0: TMA producer, MMA issuer, two idle warps; 1, 2: softmax; 3: output
constexpr int kT2Ring = 2;                   // K ring depth and V ring depth
constexpr int kT2Items = 4;                  // item descriptors in flight
constexpr int kT2MaxSeqSmem = 1024;          // sequences whose slot table fits in shared memory
constexpr float kT2Rescale = 8.0f;

static __device__ int g_status_prefill_tc2 = 0;

static __device__ unsigned int g_prefill_ticket = 0;

struct T2Item {
  int seq;        // -1: no more work
  int h;
  int q_row;      // global row of the block's first query token
  int tq0;        // that token's index within the sequence
  int Lq, Lk;
  int k_begin;    // dense K/V: first row of the sequence
  int n[2];       // K/V tiles each half needs (n[1] == 0: half B is empty)
};

// Output of one half of an item, run by the output warpgroup: read the finished O row out of TMEM
// in 32-column chunks, scale by 1 / row sum and store bf16 rows through a per-warp staging tile so
// that every store instruction writes 64-byte row segments (a thread owns a whole row: stored
// directly, each instruction would touch 32 different lines with 16 bytes each).  The accumulator
// is released as soon as its last chunk is in registers.
__device__ __forceinline__ void t2_output(const PrefillParams& p, uint32_t tmem_o_lane, uint64_t* bar_o_free,
                                          unsigned char* stage, int lane, int quarter, int hx,
                                          float inv, int q_row, int h, int tq0, int Lq) {
  const int G = p.G, QT = p.QT;
  const int srow = lane >> 1, sq = lane & 1;             // read-back role: 16 rows x 2 chunks per instruction
#pragma unroll 1
  for (int cch = 0; cch < 8; ++cch) {
    uint32_t ov[16];
    tc::ld_32x32b_x16(tmem_o_lane + cch * 16, ov);
    tc::wait_ld();
    if (cch == 7) {
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_o_free);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      uint4 w;
      w.x = pack_bf16(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
      w.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
      w.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
      w.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
      *reinterpret_cast<uint4*>(stage + lane * 32 + ((i ^ ((lane >> 2) & 1)) << 4)) = w;
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int lr = 16 * k + srow;                         // row within the warp's 32
      const uint4 w = *reinterpret_cast<const uint4*>(stage + lr * 32 + ((sq ^ ((lr >> 2) & 1)) << 4));
      const int rr = quarter * 32 + lr;                     // row of the 128-row tile
      const int tk = tq0 + hx * QT + rr / G;
      if (rr < QT * G && tk < Lq)
        *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(
            p.out + (static_cast<long long>(q_row + hx * QT + rr / G) * p.H + h * G + rr % G) * 128) +
            cch * 32 + sq * 16) = w;
    }
    __syncwarp();
  }
}

// The same for a warp whose 32 tile rows are all real query rows: the scaled bf16 rows are laid out
// in shared memory as two 128-byte-swizzled boxes of 64 dims and leave through two TMA stores, so
// the warp issues no global store and no read-back at all.  `stage` is 4 KiB, 1024-byte aligned.
__device__ __forceinline__ void t2_stage_chunk(const uint32_t (&ov)[16], unsigned char* box, int lane, int c, float inv) {
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    uint4 w;
    w.x = pack_bf16(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
    w.y = pack_bf16(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
    w.z = pack_bf16(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
    w.w = pack_bf16(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
    *reinterpret_cast<uint4*>(box + lane * 64 + (((2 * c + i) ^ ((lane >> 1) & 3)) << 4)) = w;   // 64-byte swizzle
  }
}
// `stage` holds two boxes of 32 rows x 32 dims (2 KiB each, 64-byte swizzle) used in turn, so that
// a box is written while the TMA engine still reads the one before.
__device__ __forceinline__ void t2_output_tma(const CUtensorMap* map_o, uint32_t tmem_o_lane, uint64_t* bar_o_free,
                                              unsigned char* stage, int lane, float inv, int head0, int tok0) {
  // eight 16-column chunks, the TMEM load of the next one in flight while one is converted
  uint32_t a[16], b[16];
  tc::ld_32x32b_x16(tmem_o_lane, a);
#pragma unroll
  for (int bx = 0; bx < 4; ++bx) {
    unsigned char* box = stage + (bx & 1) * 2048;
    if (lane == 0) tma_store_wait_read_but_one();        // the store before the previous one has left this box
    __syncwarp();
    tc::wait_ld();
    tc::ld_32x32b_x16(tmem_o_lane + bx * 32 + 16, b);
    t2_stage_chunk(a, box, lane, 0, inv);
    tc::wait_ld();
    if (bx == 3) {
      // the accumulator is in registers: the issuer may start the next item's PV
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_o_free);
    } else {
      tc::ld_32x32b_x16(tmem_o_lane + bx * 32 + 32, a);
    }
    t2_stage_chunk(b, box, lane, 1, inv);
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
      tma_store_3d(map_o, box, bx * 32, head0, tok0);
      tma_store_commit();
    }
  }
}

__global__ void __launch_bounds__(kT2Threads, 1)
prefill_attn_tc2_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q,
                        const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const __grid_constant__ CUtensorMap map_o) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;                              // [2][32 KiB]
  unsigned char* sK = smem + 2 * kT2Tile;                // [kT2Ring][32 KiB]
  unsigned char* sV = sK + kT2Ring * kT2Tile;            // [kT2Ring][32 KiB]
  unsigned char* sStage = sV + kT2Ring * kT2Tile;       // [8 softmax warps][32 rows x 64 B] output staging
  int* s_slot = reinterpret_cast<int*>(sStage + 8 * 2048);       // [batch + 1] first slot of every sequence
  __shared__ __align__(8) uint64_t bar_item_full[kT2Items], bar_item_empty[kT2Items];
  __shared__ __align__(8) uint64_t bar_q_full[2], bar_q_empty[2];
  __shared__ __align__(8) uint64_t bar_k_full[kT2Ring], bar_k_empty[kT2Ring], bar_v_full[kT2Ring], bar_v_empty[kT2Ring];
  __shared__ __align__(8) uint64_t bar_s_full[2], bar_p_full[2], bar_o_final[2], bar_o_free[2];
  __shared__ __align__(8) uint64_t bar_l_full[2], bar_l_empty[2];
  __shared__ float s_inv[2][128];                        // 1 / row sum of a finished half, softmax -> output warpgroup
  __shared__ __align__(16) T2Item s_item[kT2Items];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, QT = p.QT, QB = 2 * p.QT;
  const bool slot_in_smem = p.batch <= kT2MaxSeqSmem;

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < kT2Items; ++i) { mbar_init(&bar_item_full[i], 1); mbar_init(&bar_item_empty[i], 13); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bar_q_full[i], 1);
      mbar_init(&bar_q_empty[i], 1);
      mbar_init(&bar_s_full[i], 1);
      mbar_init(&bar_p_full[i], 4);
      mbar_init(&bar_o_final[i], 1);
      mbar_init(&bar_o_free[i], 4);
      mbar_init(&bar_l_full[i], 4);
      mbar_init(&bar_l_empty[i], 4);
    }
    for (int i = 0; i < kT2Ring; ++i) {
      mbar_init(&bar_k_full[i], 1);
      mbar_init(&bar_k_empty[i], 1);
      mbar_init(&bar_v_full[i], 1);
      mbar_init(&bar_v_empty[i], 1);
    }
    mbar_fence_init();
  }
  if (slot_in_smem)
    for (int i = tid; i <= p.batch; i += kT2Threads) s_slot[i] = __ldg(p.cu_q + i) / QB + i;
  if (warp == 1) {
    tc::tmem_alloc(&s_tmem_base, 512);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem_base;
  volatile int* abort_flag = &s_abort;

  // Registers move from the light warpgroup to the two softmax warpgroups, which hold a whole
  // 128-column S row (and later the O row) per thread.
  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;" ::: "memory");
  if (warp == 0) {
    // ================================ TMA producer ================================
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const unsigned int n_items = static_cast<unsigned int>(p.n_slots) * p.Hkv;
      int n_pub = 0;            // items published
      int kt = 0, vt = 0;       // K / V tiles issued so far (ring positions)
      bool ok = true;
      while (ok) {
        // a ticket; each CTA draws until it fails, the last ticket of the launch resets the counter
        const unsigned int tk = atomicAdd(&g_prefill_ticket, 1u);
        if (tk == n_items + gridDim.x - 1) atomicExch(&g_prefill_ticket, 0u);
        // the descriptor is built in its ring slot; only what the loads need stays in registers
        const int is = n_pub % kT2Items;
        if (!mbar_wait(&bar_item_empty[is], ((n_pub / kT2Items) & 1) ^ 1, abort_flag)) { ok = false; break; }
        int seq = -1, h = 0, q_row = 0, k_begin = 0, n = 0;
        bool b_rows = false;                                            // half B holds query rows
        if (tk < n_items) {
          h = tk % p.Hkv;
          const int x = p.n_slots - 1 - static_cast<int>(tk / p.Hkv);   // reverse slot order: within a sequence the later, longer blocks come first
          int lo = 0, hi = p.batch;
          while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            const int f = slot_in_smem ? s_slot[mid] : __ldg(p.cu_q + mid) / QB + mid;
            if (f <= x) lo = mid; else hi = mid;
          }
          const int q_begin = __ldg(p.cu_q + lo);
          const int Lq = __ldg(p.cu_q + lo + 1) - q_begin;
          const int qb = x - (q_begin / QB + lo);
          if (qb < 0 || qb * QB >= Lq) continue;                        // slot owns no query block
          k_begin = __ldg(p.cu_k + lo);
          const int Lk = __ldg(p.cu_k + lo + 1) - k_begin;
          const int shift = Lk - Lq;
          const int tq0 = qb * QB;
          const int nA = max(0, (min(Lk, shift + min(tq0 + QT, Lq)) + kT2Kv - 1) / kT2Kv);
          b_rows = tq0 + QT < Lq;
          const int nB = b_rows ? max(0, (min(Lk, shift + min(tq0 + QB, Lq)) + kT2Kv - 1) / kT2Kv) : 0;
          seq = lo;
          q_row = q_begin + tq0;
          n = max(nA, nB);
          s_item[is].h = h;
          s_item[is].q_row = q_row;
          s_item[is].tq0 = tq0;
          s_item[is].Lq = Lq;
          s_item[is].Lk = Lk;
          s_item[is].k_begin = k_begin;
          s_item[is].n[0] = nA;
          s_item[is].n[1] = nB;
        }
        s_item[is].seq = seq;
        mbar_arrive(&bar_item_full[is]);                                // an item, or the end marker
        if (seq < 0) break;
        // The Q tiles can only be loaded once the previous item has let go of the buffers, which is when
        // they are needed: start them on their way into L2 now, with the item's first K/V tile.
        tma_prefetch_l2_3d(&map_q, 0, h * G, q_row);
        tma_prefetch_l2_3d(&map_q, 64, h * G, q_row);
        if (b_rows) {
          tma_prefetch_l2_3d(&map_q, 0, h * G, q_row + QT);
          tma_prefetch_l2_3d(&map_q, 64, h * G, q_row + QT);
        }
        // Q tiles (the buffers are free once every S MMA of the previous item has completed)
        const uint32_t qph = (n_pub & 1) ^ 1;
        for (int hx = 0; hx < 2; ++hx) {
          if (!mbar_wait(&bar_q_empty[hx], qph, abort_flag)) { ok = false; break; }
          if (hx == 1 && !b_rows) { mbar_arrive(&bar_q_full[1]); continue; }
          mbar_expect_tx(&bar_q_full[hx], kT2Tile);
          tma_load_3d(sQ + hx * kT2Tile, &map_q, &bar_q_full[hx], 0, h * G, q_row + hx * QT);
          tma_load_3d(sQ + hx * kT2Tile + kT2Sub, &map_q, &bar_q_full[hx], 64, h * G, q_row + hx * QT);
        }
        if (!ok) break;
        ++n_pub;
        // K and V tiles
        const int* bt_row = p.block_tables ? p.block_tables + seq * p.bt_row_stride : nullptr;
        for (int j = 0; j < n; ++j) {
          int row0;
          if (bt_row) {
            const int tok0 = j * kT2Kv;
            const int col = tok0 / p.block_size;
            const long long blk = col < p.bt_cols ? bt_row[col] : -1;
            row0 = (blk >= 0 && blk < p.num_blocks) ? static_cast<int>(blk * p.block_size + (tok0 - col * p.block_size))
                                                    : -kT2Kv;
          } else {
            row0 = k_begin + j * kT2Kv;
          }
          const int ks = kt % kT2Ring;
          if (!mbar_wait(&bar_k_empty[ks], ((kt / kT2Ring) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&bar_k_full[ks], kT2Tile);
          tma_load_3d(sK + ks * kT2Tile, &map_k, &bar_k_full[ks], 0, h, row0);
          tma_load_3d(sK + ks * kT2Tile + kT2Sub, &map_k, &bar_k_full[ks], 64, h, row0);
          ++kt;
          const int vs = vt % kT2Ring;
          if (!mbar_wait(&bar_v_empty[vs], ((vt / kT2Ring) & 1) ^ 1, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&bar_v_full[vs], kT2Tile);
          tma_load_3d(sV + vs * kT2Tile, &map_v, &bar_v_full[vs], 0, h, row0);
          tma_load_3d(sV + vs * kT2Tile + kT2Sub, &map_v, &bar_v_full[vs], 64, h, row0);
          ++vt;
        }
      }
    }
  } else if (warp == 1) {
    // ================================ MMA issuer ================================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::idesc_bf16_f32(128, 128, false, false);
      constexpr uint32_t idesc_pv = tc::idesc_bf16_f32(128, 128, false, true);
      constexpr uint32_t desc_hi = tc::smem_desc_sw128_hi(1024);
      const uint32_t q_lo = tc::smem_desc_sw128_lo(smem_u32(sQ), 16), k_lo = tc::smem_desc_sw128_lo(smem_u32(sK), 16);
      const uint32_t v_lo = tc::smem_desc_sw128_lo(smem_u32(sV), kT2Sub);
      int n_item = 0, kt = 0, vt = 0;
      int np[2] = {0, 0};     // P tiles consumed per half (phase of bar_p_full)
      int no[2] = {0, 0};     // items whose O was read out per half (phase of bar_o_free)
      bool ok = true;
      auto issue_s = [&](int hx, int kslot) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = ((ks >> 2) * kT2Sub + (ks & 3) * 32) >> 4;
          tc::mma_ss_lo(tmem + hx * 128, q_lo + hx * (kT2Tile >> 4) + off, k_lo + kslot * (kT2Tile >> 4) + off, desc_hi,
                        idesc_qk, ks > 0);
        }
        tc::commit(&bar_s_full[hx]);
      };
      auto issue_pv = [&](int hx, int vslot, bool accumulate) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          tc::mma_ts_lo(tmem + 256 + hx * 128, tmem + hx * 128 + ks * 8, v_lo + vslot * (kT2Tile >> 4) + ks * (2048 >> 4),
                        desc_hi, idesc_pv, accumulate || ks > 0);
      };
      while (ok) {
        const int is = n_item % kT2Items;
        if (!mbar_wait(&bar_item_full[is], (n_item / kT2Items) & 1, abort_flag)) break;
        const int seq = s_item[is].seq, nA = s_item[is].n[0], nB = s_item[is].n[1], n = max(nA, nB);
        mbar_arrive(&bar_item_empty[is]);
        if (seq < 0) break;
        const uint32_t qph = n_item & 1;
        if (!mbar_wait(&bar_q_full[0], qph, abort_flag) || !mbar_wait(&bar_q_full[1], qph, abort_flag)) break;
        // first K tile: S for both halves
        if (n > 0) {
          if (!mbar_wait(&bar_k_full[kt % kT2Ring], (kt / kT2Ring) & 1, abort_flag)) break;
          tc::fence_after_sync();
          if (nA > 0) issue_s(0, kt % kT2Ring);
          if (nB > 0) issue_s(1, kt % kT2Ring);
          tc::commit(&bar_k_empty[kt % kT2Ring]);
          ++kt;
        }
        if (nA <= 1) tc::commit(&bar_q_empty[0]);
        if (nB <= 1) tc::commit(&bar_q_empty[1]);
        for (int j = 0; j < n && ok; ++j) {
          const int vslot = vt % kT2Ring;
          // V_j and the next K tile land long before the softmax is through: their barriers are tested
          // first, so that little but the issue itself stands between a half's P and its MMAs
          if (!mbar_wait(&bar_v_full[vslot], (vt / kT2Ring) & 1, abort_flag)) { ok = false; break; }
          if (j + 1 < n && !mbar_wait(&bar_k_full[kt % kT2Ring], (kt / kT2Ring) & 1, abort_flag)) { ok = false; break; }
          if (j == 0) {
            // the output warpgroup must have taken the previous item's O out of both accumulators
            if (nA > 0 && !mbar_wait(&bar_o_free[0], (no[0] & 1) ^ 1, abort_flag)) { ok = false; break; }
            if (nB > 0 && !mbar_wait(&bar_o_free[1], (no[1] & 1) ^ 1, abort_flag)) { ok = false; break; }
          }
          for (int hx = 0; hx < 2 && ok; ++hx) {
            const int nx = hx == 0 ? nA : nB;
            if (j >= nx) continue;
            // O_X += P_X V_j
            if (!mbar_wait(&bar_p_full[hx], np[hx] & 1, abort_flag)) { ok = false; break; }
            ++np[hx];
            tc::fence_after_sync();
            issue_pv(hx, vslot, j > 0);
            if (j == nx - 1) { tc::commit(&bar_o_final[hx]); ++no[hx]; }
            // S_X for the next K tile (its buffer is free: the PV above reads P before it runs)
            if (j + 1 < nx) {
              issue_s(hx, kt % kT2Ring);
              if (j + 2 >= nx) tc::commit(&bar_q_empty[hx]);   // that was the half's last S: its Q tile is free
            }
          }
          if (!ok) break;
          tc::commit(&bar_v_empty[vslot]);
          ++vt;
          if (j + 1 < n) { tc::commit(&bar_k_empty[kt % kT2Ring]); ++kt; }
        }
        ++n_item;
      }
    }
  }
  } else if (warp < 12) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 184;" ::: "memory");
    // ================================ softmax / epilogue ================================
    const int hx = (warp - 4) >> 2;                     // which half this warpgroup serves
    const int quarter = warp & 3;                       // TMEM lanes this warp may touch
    const int r = quarter * 32 + lane;                  // row of the (token, head) product
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tmem_s = tmem + hx * 128, tmem_o = tmem + 256 + hx * 128;
    const float c = p.scale_log2;
    int n_item = 0, ns = 0, vt_base = 0;
    bool ok = true;
    int n_fin = 0;                                      // halves handed to the output warpgroup

    while (ok) {
      const int is = n_item % kT2Items;
      if (!mbar_wait(&bar_item_full[is], (n_item / kT2Items) & 1, abort_flag)) break;
      const T2Item it = s_item[is];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_item_empty[is]);   // this warp has its copy
      if (it.seq < 0) break;
      ++n_item;
      const int nx = hx ? it.n[1] : it.n[0];
      const int n_all = max(it.n[0], it.n[1]);
      const int shift = it.Lk - it.Lq;
      const int tok = it.tq0 + hx * QT + r / G;
      const bool row_ok = r < QT * G && tok < it.Lq;
      const int kmax = row_ok ? shift + tok : -1;          // last visible key (inclusive)
      const int first_row_kmax = shift + it.tq0 + hx * QT;
      float m_used = -INFINITY, l = 0.f;
      for (int j = 0; j < nx; ++j) {
        if (!mbar_wait(&bar_s_full[hx], ns & 1, abort_flag)) { ok = false; break; }
        ++ns;
        tc::fence_after_sync();
        const int key0 = j * kT2Kv;
        const bool need_mask = key0 + kT2Kv - 1 > first_row_kmax;
        // the whole S row in registers: four TMEM loads in flight, one wait
        uint32_t sv[4][32];
#pragma unroll
        for (int cch = 0; cch < 4; ++cch) tc::ld_32x32b_x32(tmem_s + lane_base + cch * 32, sv[cch]);
        tc::wait_ld();
        if (need_mask) {
          const int nvalid = kmax - key0 + 1;           // columns of this row that may be seen
#pragma unroll
          for (int cch = 0; cch < 4; ++cch) {
            if (nvalid < (cch + 1) * 32) {              // a chunk that lies wholly below the diagonal costs nothing
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (cch * 32 + i >= nvalid) sv[cch][i] = 0xff800000u;   // -inf
            }
          }
        }
        // eight independent chains of 3-input max
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
        float mx4 = -INFINITY, mx5 = -INFINITY, mx6 = -INFINITY, mx7 = -INFINITY;
#pragma unroll
        for (int cch = 0; cch < 4; ++cch) {
#pragma unroll
          for (int i = 0; i < 32; i += 16) {
            mx0 = fmax3(mx0, __uint_as_float(sv[cch][i]), __uint_as_float(sv[cch][i + 1]));
            mx1 = fmax3(mx1, __uint_as_float(sv[cch][i + 2]), __uint_as_float(sv[cch][i + 3]));
            mx2 = fmax3(mx2, __uint_as_float(sv[cch][i + 4]), __uint_as_float(sv[cch][i + 5]));
            mx3 = fmax3(mx3, __uint_as_float(sv[cch][i + 6]), __uint_as_float(sv[cch][i + 7]));
            mx4 = fmax3(mx4, __uint_as_float(sv[cch][i + 8]), __uint_as_float(sv[cch][i + 9]));
            mx5 = fmax3(mx5, __uint_as_float(sv[cch][i + 10]), __uint_as_float(sv[cch][i + 11]));
            mx6 = fmax3(mx6, __uint_as_float(sv[cch][i + 12]), __uint_as_float(sv[cch][i + 13]));
            mx7 = fmax3(mx7, __uint_as_float(sv[cch][i + 14]), __uint_as_float(sv[cch][i + 15]));
          }
        }
        const float mx = fmax3(fmax3(mx0, mx1, mx2), fmax3(mx3, mx4, mx5), fmaxf(mx6, mx7));
        const float m_new = fmaxf(m_used, mx);
        if (j == 0) {
          m_used = m_new;
        } else {
          const bool grow = (m_new - m_used) * c > kT2Rescale;
          if (__any_sync(0xffffffffu, grow)) {
            const float alpha = grow ? fast_exp2((m_used - m_new) * c) : 1.f;
            if (grow) { m_used = m_new; l *= alpha; }
#pragma unroll
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
        // P = exp2(c * (s - m)) (masked entries are -inf -> 0), row sum, packed bf16 back over S
        const float mc = (m_used == -INFINITY ? 0.f : m_used) * c;
        // packed 2 x fp32 FMA and ADD: half the instructions of the scalar form
        const unsigned long long c2 = f32x2_pack(c, c), nmc2 = f32x2_pack(-mc, -mc);
        unsigned long long ls0 = 0ull, ls1 = 0ull, ls2 = 0ull, ls3 = 0ull;   // four independent (pair) sum chains
#pragma unroll
        for (int cch = 0; cch < 4; ++cch) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; i += 4) {
            float p0, p1, p2, p3, p4, p5, p6, p7;
            f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(sv[cch][2 * i]), __uint_as_float(sv[cch][2 * i + 1])), c2, nmc2), p0, p1);
            f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(sv[cch][2 * i + 2]), __uint_as_float(sv[cch][2 * i + 3])), c2, nmc2), p2, p3);
            f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(sv[cch][2 * i + 4]), __uint_as_float(sv[cch][2 * i + 5])), c2, nmc2), p4, p5);
            f32x2_unpack(f32x2_fma(f32x2_pack(__uint_as_float(sv[cch][2 * i + 6]), __uint_as_float(sv[cch][2 * i + 7])), c2, nmc2), p6, p7);
            p0 = fast_exp2(p0); p1 = fast_exp2(p1); p2 = fast_exp2(p2); p3 = fast_exp2(p3);
            p4 = fast_exp2(p4); p5 = fast_exp2(p5); p6 = fast_exp2(p6); p7 = fast_exp2(p7);
            ls0 = f32x2_add(ls0, f32x2_pack(p0, p1));
            ls1 = f32x2_add(ls1, f32x2_pack(p2, p3));
            ls2 = f32x2_add(ls2, f32x2_pack(p4, p5));
            ls3 = f32x2_add(ls3, f32x2_pack(p6, p7));
            pk[i] = pack_bf16(p0, p1);
            pk[i + 1] = pack_bf16(p2, p3);
            pk[i + 2] = pack_bf16(p4, p5);
            pk[i + 3] = pack_bf16(p6, p7);
          }
          tc::st_32x32b_x16(tmem_s + lane_base + cch * 16, pk);
        }
        float l0, l1, l2, l3;
        {
          float a0, a1;
          f32x2_unpack(f32x2_add(f32x2_add(ls0, ls1), f32x2_add(ls2, ls3)), a0, a1);
          l0 = a0; l1 = a1; l2 = 0.f; l3 = 0.f;
        }
        l += (l0 + l1) + (l2 + l3);
        tc::wait_st();
        if (key0 + kT2Kv > it.Lk) {
          // ragged last tile of the sequence: V rows past its end are foreign data; zero them so
          // that 0 * garbage cannot turn into NaN inside the tensor core
          const int vt = vt_base + j;
          if (!mbar_wait(&bar_v_full[vt % kT2Ring], (vt / kT2Ring) & 1, abort_flag)) { ok = false; break; }
          if (key0 + r >= it.Lk) {
            unsigned char* vrow = sV + (vt % kT2Ring) * kT2Tile + r * 128;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              *reinterpret_cast<uint4*>(vrow + i * 16) = make_uint4(0, 0, 0, 0);
              *reinterpret_cast<uint4*>(vrow + kT2Sub + i * 16) = make_uint4(0, 0, 0, 0);
            }
          }
          fence_proxy_async_smem();
        }
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_p_full[hx]);   // one arrival per warp
      }
      if (!ok) break;
      vt_base += n_all;
      if (nx > 0) {
        // the row's 1 / sum goes to the output warpgroup, which drains O while this one moves on
        if (!mbar_wait(&bar_l_empty[hx], (n_fin & 1) ^ 1, abort_flag)) { ok = false; break; }
        s_inv[hx][r] = l > 0.f ? 1.f / l : 0.f;
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_l_full[hx]);
        ++n_fin;
      } else if (row_ok) {
        // no visible key at all (Lk < Lq rows): zeros, as the reference's attention library does
        uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<long long>(it.q_row + hx * QT + r / G) * p.H + it.h * G + r % G) * 128);
#pragma unroll
        for (int i = 0; i < 16; ++i) dst[i] = make_uint4(0, 0, 0, 0);
      }
    }
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;" ::: "memory");
    // ================================ output warpgroup ================================
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    int n_item = 0;
    int nf[2] = {0, 0};                                  // halves drained so far
    bool ok = true;
    while (ok) {
      const int is = n_item % kT2Items;
      if (!mbar_wait(&bar_item_full[is], (n_item / kT2Items) & 1, abort_flag)) break;
      const int seq = s_item[is].seq, h = s_item[is].h, q_row = s_item[is].q_row, tq0 = s_item[is].tq0, Lq = s_item[is].Lq;
      const int nA = s_item[is].n[0], nB = s_item[is].n[1];
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_item_empty[is]);
      if (seq < 0) break;
      ++n_item;
#pragma unroll 1
      for (int hx = 0; hx < 2; ++hx) {
        if ((hx == 0 ? nA : nB) <= 0) continue;
        const uint32_t ph = nf[hx] & 1;
        if (!mbar_wait(&bar_l_full[hx], ph, abort_flag)) { ok = false; break; }
        const float inv = s_inv[hx][r];
        __syncwarp();
        if (lane == 0) mbar_arrive(&bar_l_empty[hx]);
        if (!mbar_wait(&bar_o_final[hx], ph, abort_flag)) { ok = false; break; }
        tc::fence_after_sync();
        const int tok_w = tq0 + hx * QT + (quarter * 32) / G;        // first token of this warp's rows
        if (p.out_tma && tok_w + 32 / G <= Lq) {
          t2_output_tma(&map_o, tmem + 256 + hx * 128 + lane_base, &bar_o_free[hx], sStage + quarter * 4096, lane, inv,
                        h * G, q_row + hx * QT + (quarter * 32) / G);
        } else {
          if (lane == 0) tma_store_wait_read();
          __syncwarp();
          t2_output(p, tmem + 256 + hx * 128 + lane_base, &bar_o_free[hx], sStage + quarter * 4096, lane, quarter, hx,
                    inv, q_row, h, tq0, Lq);
        }
        ++nf[hx];
      }
    }
    if (lane == 0) tma_store_wait_read();                // the staging tile must outlive its last store
  }

  // ---- teardown: everyone meets, then the allocating warp frees TMEM ----
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, 512);
  }
  if (tid == 0 && s_abort) atomicExch(&g_status_prefill_tc2, 1);
}


int read_status_prefill_tc2() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_status_prefill_tc2, sizeof(int));
  return v;
}

// A launch that gave up on a wait never draws its last ticket, so the counter keeps a stale value that
// would make the next launch skip its first items: clear it together with the status word.
int reset_state_prefill_tc2() {
  const int zero = 0;
  const unsigned int uzero = 0;
  int rc = check_cuda(cudaMemcpyToSymbol(g_status_prefill_tc2, &zero, sizeof(int)), "device_status: clearing the tcgen05 status word");
  if (rc) return rc;
  return check_cuda(cudaMemcpyToSymbol(g_prefill_ticket, &uzero, sizeof(unsigned int)), "device_status: clearing the ticket counter");
}

int inject_timeout_prefill_tc2() {
  const int one = 1;
  const unsigned int stale = 7;
  int rc = check_cuda(cudaMemcpyToSymbol(g_status_prefill_tc2, &one, sizeof(int)), "inject_timeout: status word");
  if (rc) return rc;
  return check_cuda(cudaMemcpyToSymbol(g_prefill_ticket, &stale, sizeof(unsigned int)), "inject_timeout: ticket counter");
}

// Needs whole query heads groups in a 128-row tile.  The query-block slots are laid out for 2 * QT tokens.
int launch_prefill_tc2(PrefillParams p, const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                       const CUtensorMap& map_o, cudaStream_t stream) {
  p.n_slots = p.total_q / (2 * p.QT) + p.batch;
  const size_t smem = 1024 + static_cast<size_t>(2 + 2 * kT2Ring) * kT2Tile + 8 * 2048 +
                      (p.batch <= kT2MaxSeqSmem ? (p.batch + 1) * 4 : 4) + 64;
  static std::atomic<size_t> configured[kMaxDevices];
  const int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(prefill_attn_tc2_kernel), smem, configured,
                                     "prefill_attn(tcgen05): cudaFuncSetAttribute");
  if (rc) return rc;
  const int grid = sm_count();
  if (grid <= 0) return set_error(kErrNoDriver, "prefill_attn: no CUDA device");
  if (static_cast<long long>(p.n_slots) * p.Hkv > 0x7fffffffLL) return set_error(kErrBadShape, "prefill_attn: too many query blocks");
  prefill_attn_tc2_kernel<<<grid, kT2Threads, smem, stream>>>(p, map_q, map_k, map_v, map_o);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "prefill_attn(tc2) launch");
}

}  // namespace b200
