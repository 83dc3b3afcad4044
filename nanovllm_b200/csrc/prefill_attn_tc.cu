// Varlen causal prefill attention on the 5th-generation tensor cores (tcgen05.mma with TMEM
// accumulators), for dense K/V and for K/V read from the paged cache.  Replaces
// flash_attn_varlen_func as called at nanovllm/layers/attention.py:64-70.
//
// One CTA owns 128 rows = (128 / G query tokens) x (the G query heads of one kv head), so each
// K/V tile is fetched once for all query heads that share it.  Roles:
//   warp 0      TMA producer: the Q tile once, then one 128-token K tile and V tile per step
//               (two 64-column boxes each, 128-byte swizzle, the canonical UMMA operand layout);
//   warp 1      one elected thread issues tcgen05.mma: S = Q K^T (M128 N128, 8 k-steps of 16) into
//               TMEM columns [0,128), then O += P V (A = P read from TMEM, B = V as an MN-major
//               shared-memory operand) into TMEM columns [128,256);
//   warps 2-5   softmax: thread r owns TMEM lane r = one row.  It reads its S row with tcgen05.ld,
//               keeps the running max and sum in registers (no shuffles: a row never leaves its
//               thread), writes P as packed bf16 back over S with tcgen05.st, and rescales O in
//               TMEM only when the row maximum has grown by more than 2^8 (lazy rescaling).
// TMEM use is 256 columns per CTA, so two CTAs share an SM and their MMA / exp phases interleave.
// Every mbarrier wait is bounded; on a timeout all roles unwind, TMEM is freed, a status word is set.
#include <atomic>

#include "../../include/b200_attn.h"
#include "kernels.cuh"
#include "tcgen05.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kTcKv = 128;                 // keys per step
constexpr int kTcSub = 128 * 128;          // one 64-column sub-tile of a 128-row tile (bytes)
constexpr int kTcTileBytes = 2 * kTcSub;   // 128 rows x 128 dims bf16
constexpr int kTcThreads = 192;
constexpr uint32_t kTcTmemCols = 256;
constexpr float kRescaleThreshold = 8.0f;  // log2 domain

static __device__ int g_status_prefill_tc = 0;

__global__ void __launch_bounds__(kTcThreads, 2)
prefill_attn_tc_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_q,
                       const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;
  unsigned char* sK = smem + kTcTileBytes;
  unsigned char* sV = smem + 2 * kTcTileBytes;
  __shared__ __align__(8) uint64_t bar_q_full, bar_k_full, bar_k_empty, bar_v_full, bar_v_empty, bar_s_full, bar_p_full,
      bar_o_final;
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, QT = p.QT;
  const int h = blockIdx.x % p.Hkv;
  const int x = p.n_slots - 1 - static_cast<int>(blockIdx.x / p.Hkv);  // later (heavier) tiles first

  // slot -> (sequence, query tile); identical to the mma.sync variant
  int lo = 0, hi = p.batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (__ldg(p.cu_q + mid) / QT + mid <= x) lo = mid; else hi = mid;
  }
  const int seq = lo;
  const int q_begin = __ldg(p.cu_q + seq), q_end = __ldg(p.cu_q + seq + 1);
  const int Lq = q_end - q_begin;
  const int qt = x - (q_begin / QT + seq);
  if (qt < 0 || qt * QT >= Lq) return;
  const int k_begin = __ldg(p.cu_k + seq);
  const int Lk = __ldg(p.cu_k + seq + 1) - k_begin;
  const int tq0 = qt * QT;
  const int tq1 = min(tq0 + QT, Lq);
  const int shift = Lk - Lq;
  const int kv_end = min(Lk, shift + tq1);
  const int n_tiles = (kv_end + kTcKv - 1) / kTcKv;
  if (n_tiles <= 0) {
    for (int e = tid; e < (tq1 - tq0) * G * 128; e += kTcThreads) {
      const int r = e >> 7, d = e & 127;
      p.out[(static_cast<long long>(q_begin + tq0 + r / G) * p.H + h * G + r % G) * 128 + d] = __float2bfloat16(0.f);
    }
    return;
  }

  if (tid == 0) {
    s_abort = 0;
    mbar_init(&bar_q_full, 1);
    mbar_init(&bar_k_full, 1);
    mbar_init(&bar_k_empty, 1);
    mbar_init(&bar_v_full, 1);
    mbar_init(&bar_v_empty, 1);
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_p_full, 128);
    mbar_init(&bar_o_final, 1);
    mbar_fence_init();
  }
  if (warp == 1) {
    tc::tmem_alloc(&s_tmem_base, kTcTmemCols);
    tc::tmem_relinquish();
  }
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem_base;
  const uint32_t tmem_s = tmem;         // S (fp32, 128 columns); P (bf16 pairs) overwrites columns [0,64)
  const uint32_t tmem_o = tmem + 128;   // O (fp32, 128 columns)
  volatile int* abort_flag = &s_abort;

  if (warp == 0) {
    // ============================ TMA producer ============================
    if (lane == 0) {
      tma_prefetch_desc(&map_q);
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      mbar_expect_tx(&bar_q_full, kTcTileBytes);
      tma_load_3d(sQ, &map_q, &bar_q_full, 0, h * G, q_begin + tq0);
      tma_load_3d(sQ + kTcSub, &map_q, &bar_q_full, 64, h * G, q_begin + tq0);
      const int* bt_row = p.block_tables ? p.block_tables + seq * p.bt_row_stride : nullptr;
      for (int j = 0; j < n_tiles; ++j) {
        int row0;
        if (bt_row) {
          const int tok0 = j * kTcKv;
          const int col = tok0 / p.block_size;
          const long long blk = col < p.bt_cols ? bt_row[col] : -1;
          row0 = (blk >= 0 && blk < p.num_blocks) ? static_cast<int>(blk * p.block_size + (tok0 - col * p.block_size))
                                                  : -kTcKv;
        } else {
          row0 = k_begin + j * kTcKv;
        }
        const uint32_t ph = j & 1;
        if (!mbar_wait(&bar_k_empty, ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&bar_k_full, kTcTileBytes);
        tma_load_3d(sK, &map_k, &bar_k_full, 0, h, row0);
        tma_load_3d(sK + kTcSub, &map_k, &bar_k_full, 64, h, row0);
        if (!mbar_wait(&bar_v_empty, ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&bar_v_full, kTcTileBytes);
        tma_load_3d(sV, &map_v, &bar_v_full, 0, h, row0);
        tma_load_3d(sV + kTcSub, &map_v, &bar_v_full, 64, h, row0);
      }
    }
  } else if (warp == 1) {
    // ============================ MMA issuer ============================
    if (lane == 0) {
      constexpr uint32_t idesc_qk = tc::idesc_bf16_f32(128, 128, false, false);
      constexpr uint32_t idesc_pv = tc::idesc_bf16_f32(128, 128, false, true);
      const uint32_t q_addr = smem_u32(sQ), k_addr = smem_u32(sK), v_addr = smem_u32(sV);
      bool ok = mbar_wait(&bar_q_full, 0, abort_flag);
      for (int j = 0; j < n_tiles && ok; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(&bar_k_full, ph, abort_flag)) break;
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * kTcSub + (ks & 3) * 32;
          tc::mma_ss(tmem_s, tc::smem_desc_sw128(q_addr + off, 16, 1024), tc::smem_desc_sw128(k_addr + off, 16, 1024),
                     idesc_qk, ks > 0);
        }
        tc::commit(&bar_s_full);
        tc::commit(&bar_k_empty);
        if (!mbar_wait(&bar_p_full, ph, abort_flag)) break;
        if (!mbar_wait(&bar_v_full, ph, abort_flag)) break;
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          // A: 16 keys of P = 8 packed columns; B: 16 key rows of V (2048 bytes), both 64-dim halves
          tc::mma_ts(tmem_o, tmem_s + ks * 8, tc::smem_desc_sw128(v_addr + ks * 2048, kTcSub, 1024), idesc_pv,
                     j > 0 || ks > 0);
        }
        tc::commit(&bar_v_empty);
        if (j == n_tiles - 1) tc::commit(&bar_o_final);
      }
    }
  } else {
    // ============================ softmax / epilogue ============================
    const int quarter = warp & 3;                       // TMEM lanes this warp may touch: 32*quarter ..
    const int r = quarter * 32 + lane;                  // row of the (token, head) product
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const int tok = tq0 + r / G;
    const bool row_ok = r < QT * G && tok < Lq;
    const int kmax = row_ok ? shift + tok : -1;          // last visible key (inclusive)
    const float c = p.scale_log2;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles; ++j) {
      const uint32_t ph = j & 1;
      if (!mbar_wait(&bar_s_full, ph, abort_flag)) { ok = false; break; }
      tc::fence_after_sync();
      const int key0 = j * kTcKv;
      const bool need_mask = key0 + kTcKv - 1 > shift + tq0;   // some row of the tile cannot see every key
      // ---- pass 1: row maximum ----
      float mx = -INFINITY;
#pragma unroll
      for (int cch = 0; cch < 4; ++cch) {
        uint32_t v[32];
        tc::ld_32x32b_x32(tmem_s + lane_base + cch * 32, v);
        tc::wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float s = __uint_as_float(v[i]);
          if (need_mask && key0 + cch * 32 + i > kmax) s = -INFINITY;
          mx = fmaxf(mx, s);
        }
      }
      const float m_new = fmaxf(m_used, mx);
      if (j == 0) {
        m_used = m_new;
      } else {
        const bool grow = (m_new - m_used) * c > kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = grow ? fast_exp2((m_used - m_new) * c) : 1.f;
          if (grow) { m_used = m_new; l *= alpha; }
#pragma unroll
          for (int cch = 0; cch < 4; ++cch) {
            uint32_t v[32];
            tc::ld_32x32b_x32(tmem_o + lane_base + cch * 32, v);
            tc::wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tc::st_32x32b_x32(tmem_o + lane_base + cch * 32, v);
          }
        }
      }
      // ---- pass 2: P = exp2(c * (s - m)), row sum, packed bf16 back over S ----
      const float mc = (m_used == -INFINITY ? 0.f : m_used) * c;
#pragma unroll
      for (int cch = 0; cch < 4; ++cch) {
        uint32_t v[32];
        tc::ld_32x32b_x32(tmem_s + lane_base + cch * 32, v);
        tc::wait_ld();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float p0 = fast_exp2(fmaf(__uint_as_float(v[2 * i]), c, -mc));
          float p1 = fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), c, -mc));
          if (need_mask) {
            if (key0 + cch * 32 + 2 * i > kmax) p0 = 0.f;
            if (key0 + cch * 32 + 2 * i + 1 > kmax) p1 = 0.f;
          }
          l += p0 + p1;
          pk[i] = pack_bf16(p0, p1);
        }
        tc::st_32x32b_x16(tmem_s + lane_base + cch * 16, pk);
      }
      tc::wait_st();
      if (key0 + kTcKv > Lk) {
        // last, ragged tile: V rows past the sequence end are foreign data; zero them so that
        // 0 * garbage cannot turn into NaN inside the tensor core
        if (!mbar_wait(&bar_v_full, ph, abort_flag)) { ok = false; break; }
        if (key0 + r >= Lk) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            *reinterpret_cast<uint4*>(sV + r * 128 + i * 16) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(sV + kTcSub + r * 128 + i * 16) = make_uint4(0, 0, 0, 0);
          }
        }
        fence_proxy_async_smem();
      }
      tc::fence_before_sync();
      mbar_arrive(&bar_p_full);
    }
    if (ok && mbar_wait(&bar_o_final, 0, abort_flag)) {
      tc::fence_after_sync();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(p.out + (static_cast<long long>(q_begin + tok) * p.H + h * G + r % G) * 128);
#pragma unroll
      for (int cch = 0; cch < 4; ++cch) {
        uint32_t v[32];
        tc::ld_32x32b_x32(tmem_o + lane_base + cch * 32, v);
        tc::wait_ld();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[8 * i]) * inv, __uint_as_float(v[8 * i + 1]) * inv);
            w.y = pack_bf16(__uint_as_float(v[8 * i + 2]) * inv, __uint_as_float(v[8 * i + 3]) * inv);
            w.z = pack_bf16(__uint_as_float(v[8 * i + 4]) * inv, __uint_as_float(v[8 * i + 5]) * inv);
            w.w = pack_bf16(__uint_as_float(v[8 * i + 6]) * inv, __uint_as_float(v[8 * i + 7]) * inv);
            dst[cch * 4 + i] = w;
          }
        }
      }
    }
  }

  // ---- teardown: everyone meets, then the allocating warp frees TMEM ----
  tc::fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc::fence_after_sync();
    tc::tmem_dealloc(tmem, kTcTmemCols);
  }
  if (tid == 0 && s_abort) atomicExch(&g_status_prefill_tc, 1);
}

int read_status_prefill_tc() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_status_prefill_tc, sizeof(int));
  return v;
}

bool prefill_tc_supports(const PrefillParams& p) { return p.G >= 1 && p.G <= 128 && 128 % p.G == 0; }

int launch_prefill_tc(const PrefillParams& p, const CUtensorMap& map_q, const CUtensorMap& map_k,
                      const CUtensorMap& map_v, cudaStream_t stream) {
  const size_t smem = 1024 + 3 * static_cast<size_t>(kTcTileBytes);
  static std::atomic<int> configured{0};
  if (!configured.load()) {
    int rc = check_cuda(cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                        "prefill_attn(tc): cudaFuncSetAttribute");
    if (rc) return rc;
    configured.store(1);
  }
  const long long blocks = static_cast<long long>(p.n_slots) * p.Hkv;
  if (blocks <= 0) return kOk;
  if (blocks > 0x7fffffffLL) return set_error(kErrBadShape, "prefill_attn: too many query tiles");
  prefill_attn_tc_kernel<<<static_cast<unsigned>(blocks), kTcThreads, smem, stream>>>(p, map_q, map_k, map_v);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "prefill_attn(tc) launch");
}

}  // namespace b200
