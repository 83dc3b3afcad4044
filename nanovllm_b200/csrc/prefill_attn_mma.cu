// Varlen causal prefill attention on warp-level mma.sync (the portable variant; the tcgen05
// kernel in prefill_attn_tc.cu is the fast path).  Replaces flash_attn_varlen_func as called at
// nanovllm/layers/attention.py:64-70, for dense K/V and for K/V read from the paged cache.
//
// One CTA owns `QT = 128 / G` consecutive query tokens of one sequence for one kv head: its
// 16-row-per-warp M dimension is the (token, query-head-of-the-group) product, so each K/V tile
// is loaded once for all G query heads that share it.  K/V arrive as 64-token TMA tiles through
// a 4-stage mbarrier ring fed by a producer warp; 8 consumer warps run QK^T, online softmax and
// PV in registers.
#include <atomic>

#include "../../include/b200_attn.h"
#include "kernels.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kPfTile = 64;
constexpr int kPfSub = kPfTile * 128;
constexpr int kPfStageBytes = 4 * kPfSub;
constexpr int kPfStages = 4;
constexpr int kPfConsumerWarps = 8;
constexpr int kPfConsumers = kPfConsumerWarps * 32;
constexpr int kPfThreads = kPfConsumers + 32;

static __device__ int g_status_prefill_mma = 0;

__global__ void __launch_bounds__(kPfThreads, 1)
prefill_attn_mma_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* stages = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t bar_full[kPfStages];
  __shared__ __align__(8) uint64_t bar_empty[kPfStages];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, QT = p.QT;
  const int h = blockIdx.x % p.Hkv;
  const int x = p.n_slots - 1 - static_cast<int>(blockIdx.x / p.Hkv);  // later (heavier) tiles first

  // slot -> (sequence, query tile): sequence i owns slots [cu_q[i] / QT + i, ... + ceil(Lq_i / QT))
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
  const int tq0 = qt * QT;                       // first query token of this CTA within the sequence
  const int tq1 = min(tq0 + QT, Lq);
  const int shift = Lk - Lq;                     // bottom-right causal alignment
  const int kv_end = min(Lk, shift + tq1);       // keys [0, kv_end) are visible to at least one row
  const int n_tiles = (kv_end + kPfTile - 1) / kPfTile;
  if (n_tiles <= 0) {
    // no visible key (Lk < Lq rows): zeros, as the reference's attention library does
    for (int e = tid; e < (tq1 - tq0) * G * 128; e += kPfThreads) {
      const int r = e >> 7, d = e & 127;
      p.out[(static_cast<long long>(q_begin + tq0 + r / G) * p.H + h * G + r % G) * 128 + d] = __float2bfloat16(0.f);
    }
    return;
  }

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], kPfConsumerWarps);
    }
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* abort_flag = &s_abort;

  if (warp == kPfConsumerWarps) {
    if (lane == 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      const int* bt_row = p.block_tables ? p.block_tables + seq * p.bt_row_stride : nullptr;
      for (int t = 0; t < n_tiles; ++t) {
        const int stage = t % kPfStages;
        const uint32_t ph = (t / kPfStages) & 1;
        if (!mbar_wait(&bar_empty[stage], ph ^ 1, abort_flag)) { atomicExch(&g_status_prefill_mma, 1); break; }
        int row0;
        if (bt_row) {
          const int tok0 = t * kPfTile;
          const int col = tok0 / p.block_size;
          const long long blk = col < p.bt_cols ? bt_row[col] : -1;
          row0 = (blk >= 0 && blk < p.num_blocks) ? static_cast<int>(blk * p.block_size + (tok0 - col * p.block_size))
                                                  : -kPfTile;
        } else {
          row0 = k_begin + t * kPfTile;
        }
        unsigned char* st = stages + stage * kPfStageBytes;
        mbar_expect_tx(&bar_full[stage], kPfStageBytes);
        tma_load_3d(st, &map_k, &bar_full[stage], 0, h, row0);
        tma_load_3d(st + kPfSub, &map_k, &bar_full[stage], 64, h, row0);
        tma_load_3d(st + 2 * kPfSub, &map_v, &bar_full[stage], 0, h, row0);
        tma_load_3d(st + 3 * kPfSub, &map_v, &bar_full[stage], 64, h, row0);
      }
    }
    return;
  }

  // ------------------------------- consumers -------------------------------
  const int quad = lane & 3;
  const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;      // rows of the (token, head) product
  const int tok0 = tq0 + r0 / G, tok1 = tq0 + r1 / G;       // query token within the sequence
  const bool ok0 = r0 < QT * G && tok0 < Lq, ok1 = r1 < QT * G && tok1 < Lq;
  const int kmax0 = ok0 ? shift + tok0 : -1;                // last visible key (inclusive)
  const int kmax1 = ok1 ? shift + tok1 : -1;
  int wmax = max(kmax0, kmax1), wmin = min(kmax0, kmax1);
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    wmax = max(wmax, __shfl_xor_sync(0xffffffffu, wmax, off));
    wmin = min(wmin, __shfl_xor_sync(0xffffffffu, wmin, off));
  }

  uint32_t qa[8][4];
  {
    const uint32_t* q0 = reinterpret_cast<const uint32_t*>(
        p.q + static_cast<long long>(q_begin + tok0) * p.q_row_stride + (h * G + r0 % G) * 128);
    const uint32_t* q1 = reinterpret_cast<const uint32_t*>(
        p.q + static_cast<long long>(q_begin + tok1) * p.q_row_stride + (h * G + r1 % G) * 128);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = ok0 ? __ldg(q0 + ks * 8 + quad) : 0u;
      qa[ks][1] = ok1 ? __ldg(q1 + ks * 8 + quad) : 0u;
      qa[ks][2] = ok0 ? __ldg(q0 + ks * 8 + 4 + quad) : 0u;
      qa[ks][3] = ok1 ? __ldg(q1 + ks * 8 + 4 + quad) : 0u;
    }
  }
  float o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const int stage = t % kPfStages;
    const uint32_t ph = (t / kPfStages) & 1;
    if (!mbar_wait(&bar_full[stage], ph, abort_flag)) { if (lane == 0) atomicExch(&g_status_prefill_mma, 1); return; }
    const int key0 = t * kPfTile;
    if (key0 + kPfTile > Lk) {
      // ragged last tile: rows past the sequence end are foreign data; zero V there
      unsigned char* vb = stages + stage * kPfStageBytes + 2 * kPfSub;
      const int first = Lk - key0;
      for (int e = tid; e < (kPfTile - first) * 16; e += kPfConsumers) {
        const int r = first + (e >> 4), c = e & 15;
        *reinterpret_cast<uint4*>(vb + (c >> 3) * kPfSub + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = make_uint4(0, 0, 0, 0);
      }
      fence_proxy_async_smem();
      named_bar_sync(1, kPfConsumers);
    }
    if (key0 <= wmax) {
      const uint32_t st = smem_u32(stages + stage * kPfStageBytes);
      const uint32_t k_base = st, v_base = st + 2 * kPfSub;
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      {
        const int trow = ((lane >> 4) << 3) + (lane & 7);
        const int dsel = ((lane >> 3) & 1) << 3;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
          for (int j2 = 0; j2 < 4; ++j2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + tile_offset(j2 * 16 + trow, ks * 16 + dsel, kPfTile), b0, b1, b2, b3);
            mma_bf16_16816(s[2 * j2], qa[ks], b0, b1);
            mma_bf16_16816(s[2 * j2 + 1], qa[ks], b2, b3);
          }
        }
      }
      const bool need_mask = key0 + kPfTile - 1 > wmin;
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int key = key0 + j * 8 + quad * 2 + e;
          float v0 = s[j][e] * p.scale_log2, v1 = s[j][2 + e] * p.scale_log2;
          if (need_mask) {
            if (key > kmax0) v0 = -INFINITY;
            if (key > kmax1) v1 = -INFINITY;
          }
          s[j][e] = v0;
          s[j][2 + e] = v1;
          mx0 = fmaxf(mx0, v0);
          mx1 = fmaxf(mx1, v1);
        }
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
      const float a0 = fast_exp2(m0 - ms0), a1 = fast_exp2(m1 - ms1);
      m0 = mn0; m1 = mn1;
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          s[j][e] = fast_exp2(s[j][e] - ms0);
          s[j][2 + e] = fast_exp2(s[j][2 + e] - ms1);
          ps0 += s[j][e];
          ps1 += s[j][2 + e];
        }
      }
      l0 = l0 * a0 + ps0;
      l1 = l1 * a1 + ps1;
      if (a0 != 1.f || a1 != 1.f) {
#pragma unroll
        for (int n = 0; n < 16; ++n) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
      }
      {
        const int trow = (((lane >> 3) & 1) << 3) + (lane & 7);
        const int dsel = (lane >> 4) << 3;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          uint32_t pa[4];
          pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
          pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
          pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
          pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
          for (int n2 = 0; n2 < 8; ++n2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_base + tile_offset(kk * 16 + trow, n2 * 16 + dsel, kPfTile), b0, b1, b2, b3);
            mma_bf16_16816(o[2 * n2], pa, b0, b1);
            mma_bf16_16816(o[2 * n2 + 1], pa, b2, b3);
          }
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&bar_empty[stage]);
  }

  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  if (ok0) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (static_cast<long long>(q_begin + tok0) * p.H + h * G + r0 % G) * 128);
#pragma unroll
    for (int n = 0; n < 16; ++n) dst[n * 4 + quad] = pack_bf16(o[n][0] * inv0, o[n][1] * inv0);
  }
  if (ok1) {
    uint32_t* dst = reinterpret_cast<uint32_t*>(p.out + (static_cast<long long>(q_begin + tok1) * p.H + h * G + r1 % G) * 128);
#pragma unroll
    for (int n = 0; n < 16; ++n) dst[n * 4 + quad] = pack_bf16(o[n][2] * inv1, o[n][3] * inv1);
  }
}

int launch_prefill_mma(const PrefillParams& p, const CUtensorMap& map_k, const CUtensorMap& map_v, cudaStream_t stream) {
  const size_t smem = 1024 + static_cast<size_t>(kPfStages) * kPfStageBytes;
  static std::atomic<size_t> configured[kMaxDevices];
  const int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(prefill_attn_mma_kernel), smem, configured,
                                     "prefill_attn(mma.sync): cudaFuncSetAttribute");
  if (rc) return rc;
  const long long blocks = static_cast<long long>(p.n_slots) * p.Hkv;
  if (blocks <= 0) return kOk;
  if (blocks > 0x7fffffffLL) return set_error(kErrBadShape, "prefill_attn: too many query tiles");
  prefill_attn_mma_kernel<<<static_cast<unsigned>(blocks), kPfThreads, smem, stream>>>(p, map_k, map_v);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "prefill_attn launch");
}

int read_status_prefill_mma() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_status_prefill_mma, sizeof(int));
  return v;
}

int reset_state_prefill_mma() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_status_prefill_mma, &zero, sizeof(int)), "device_status: clearing the mma.sync status word");
}

}  // namespace b200
