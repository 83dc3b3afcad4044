// Paged single-token decode attention (replaces flash_attn_with_kvcache as called at
// nanovllm/layers/attention.py:71-74).
//
// HBM-bound: every K and V byte of every context token is read exactly once.  Design:
//  * Work unit = one 64-token tile of one (sequence, kv head).  The tiles of all sequences and
//    heads form one flat list; the persistent grid (2 CTAs per SM) cuts that list into equal
//    contiguous ranges, so every CTA streams the same number of bytes whatever the length
//    distribution.  The list is derived on the device from context_lens (a block scan per CTA):
//    the launch geometry never depends on device data, as CUDA-graph replay requires.
//  * A producer warp walks the range and issues TMA tile loads (two 64x64 boxes for K, two for
//    V, 128-byte swizzle) into a ring of shared-memory stages guarded by full/empty mbarriers;
//    the ring never drains at sequence boundaries.
//  * Four consumer warps take 16 tokens of each tile: QK^T and PV on mma.sync.m16n8k16 (the G
//    query heads of the kv head are rows of the 16-row A operand), online softmax in fp32 with
//    quad shuffles, then a cross-warp combine in shared memory.
//  * A (sequence, head) cut by range boundaries leaves per-CTA partials (m, l, unnormalised O) in
//    the workspace; the last CTA to arrive (one atomic counter per (sequence, head), reset by that
//    CTA) merges them.  No CTA ever waits for another.
#include <atomic>

#include "../../include/b200_attn.h"
#include "kernels.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kTile = 64;                       // tokens per stage
constexpr int kSubTileBytes = kTile * 128;      // 64 tokens x 64 dims bf16
constexpr int kStageBytes = 4 * kSubTileBytes;  // K lo, K hi, V lo, V hi
constexpr int kDecStages = 3;
constexpr int kDecConsumerWarps = 4;
constexpr int kDecConsumers = kDecConsumerWarps * 32;
constexpr int kDecThreads = kDecConsumers + 32;
constexpr int kDecMaxBatch = 1024;              // per launch; the host splits larger batches
constexpr int kDecPer = (kDecMaxBatch + kDecThreads - 1) / kDecThreads;
constexpr int kMaxG = 16;
constexpr int kWsStatusBytes = 256;  // reserved header
static __device__ int g_status_decode = 0;

struct DecodeParams {
  const __nv_bfloat16* q;
  long long q_row_stride;
  __nv_bfloat16* out;
  const int* context_lens;
  const int* block_tables;
  long long bt_row_stride;
  int bt_cols;
  int batch, H, Hkv, G;
  int block_size;
  long long num_blocks;
  float scale_log2;
  float* ws_o;    // [2 * grid][G][128] unnormalised partial outputs
  float* ws_ml;   // [2 * grid][G][2]   running max (log2 domain) and sum
  int* counters;  // [batch * Hkv], zero between launches
};

__device__ __forceinline__ int dec_merge_floats(int G) { return kDecConsumerWarps * G * 128; }

__global__ void __launch_bounds__(kDecThreads, 2)
decode_attn_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* stages = smem;
  float* merge_o = reinterpret_cast<float*>(smem + kDecStages * kStageBytes);
  float* merge_ml = merge_o + dec_merge_floats(p.G);
  int* s_prefix = reinterpret_cast<int*>(merge_ml + kDecConsumerWarps * p.G * 2);
  __shared__ __align__(8) uint64_t bar_full[kDecStages];
  __shared__ __align__(8) uint64_t bar_empty[kDecStages];
  __shared__ int s_warp_sums[kDecThreads / 32];
  __shared__ int s_abort;
  __shared__ int s_last;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = p.G, Hkv = p.Hkv;
  const int max_len = p.bt_cols * p.block_size;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], kDecConsumerWarps);
    }
    mbar_fence_init();
  }

  // ---- tile counts per sequence and their exclusive prefix (block scan) ----
  {
    const int per = (p.batch + kDecThreads - 1) / kDecThreads;
    const int i0 = tid * per;
    int local[kDecPer];
    int sum = 0;
#pragma unroll
    for (int k = 0; k < kDecPer; ++k) {
      int nt = 0;
      const int i = i0 + k;
      if (k < per && i < p.batch) {
        int len = p.context_lens[i];
        len = len < 0 ? 0 : (len > max_len ? max_len : len);
        nt = (len + kTile - 1) / kTile;
      }
      local[k] = nt;
      sum += nt;
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) s_warp_sums[warp] = incl;
    __syncthreads();
    int excl = incl - sum;
    for (int w = 0; w < warp; ++w) excl += s_warp_sums[w];
#pragma unroll
    for (int k = 0; k < kDecPer; ++k) {
      const int i = i0 + k;
      if (k < per && i < p.batch) {
        s_prefix[i] = excl;
        excl += local[k];
        if (i == p.batch - 1) s_prefix[p.batch] = excl;
      }
    }
    __syncthreads();
  }

  // ---- sequences with no context produce zeros ----
  for (int i = blockIdx.x; i < p.batch; i += gridDim.x) {
    if (s_prefix[i + 1] == s_prefix[i]) {
      uint4* o = reinterpret_cast<uint4*>(p.out + static_cast<long long>(i) * p.H * 128);
      for (int v = tid; v < p.H * 16; v += kDecThreads) o[v] = make_uint4(0, 0, 0, 0);
    }
  }

  const long long T = static_cast<long long>(s_prefix[p.batch]) * Hkv;  // tile units in this launch
  const long long grid_eff = T < gridDim.x ? T : gridDim.x;
  const long long cta = blockIdx.x;
  if (cta >= grid_eff) return;
  const long long r_begin = cta * T / grid_eff;
  const long long r_end = (cta + 1) * T / grid_eff;

  volatile int* abort_flag = &s_abort;

  if (warp == kDecConsumerWarps) {
    // =========================== producer warp ===========================
    if (lane == 0) {
      tma_prefetch_desc(&map_k);
      tma_prefetch_desc(&map_v);
      int it = 0;
      long long x = r_begin;
      bool ok = true;
      while (x < r_end && ok) {
        int lo = 0, hi = p.batch;
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (static_cast<long long>(s_prefix[mid]) * Hkv <= x) lo = mid; else hi = mid;
        }
        const int seq = lo;
        const int nt = s_prefix[seq + 1] - s_prefix[seq];
        const long long rem = x - static_cast<long long>(s_prefix[seq]) * Hkv;
        const int h = static_cast<int>(rem / nt);
        const int t0 = static_cast<int>(rem - static_cast<long long>(h) * nt);
        const long long seg_end = x - t0 + nt;
        const long long my_end = seg_end < r_end ? seg_end : r_end;
        const int t1 = t0 + static_cast<int>(my_end - x);
        const int* bt_row = p.block_tables + seq * p.bt_row_stride;
        int cur_col = -1;
        long long cur_block = -1;
        for (int t = t0; t < t1; ++t, ++it) {
          const int stage = it % kDecStages;
          const uint32_t ph = (it / kDecStages) & 1;
          if (!mbar_wait(&bar_empty[stage], ph ^ 1, abort_flag)) { ok = false; break; }
          const int tok0 = t * kTile;
          const int col = tok0 / p.block_size;
          if (col != cur_col) { cur_col = col; cur_block = bt_row[col]; }
          int slot0 = -kTile;  // out-of-range block id: the box lies outside the tensor and reads zeros
          if (cur_block >= 0 && cur_block < p.num_blocks)
            slot0 = static_cast<int>(cur_block * p.block_size + (tok0 - col * p.block_size));
          unsigned char* st = stages + stage * kStageBytes;
          mbar_expect_tx(&bar_full[stage], kStageBytes);
          tma_load_3d(st, &map_k, &bar_full[stage], 0, h, slot0);
          tma_load_3d(st + kSubTileBytes, &map_k, &bar_full[stage], 64, h, slot0);
          tma_load_3d(st + 2 * kSubTileBytes, &map_v, &bar_full[stage], 0, h, slot0);
          tma_load_3d(st + 3 * kSubTileBytes, &map_v, &bar_full[stage], 64, h, slot0);
        }
        x = my_end;
      }
      if (!ok) {
        // unwind: give loads already issued a bounded chance to land before the CTA exits
        atomicExch(&g_status_decode, 1);
      }
    }
    return;
  }

  // ============================= consumer warps =============================
  const int row = lane >> 2;        // A/C fragment row (query head within the kv group)
  const int quad = lane & 3;
  const bool row0_ok = row < G, row1_ok = row + 8 < G;
  int it = 0;
  long long x = r_begin;
  bool ok = true;
  while (x < r_end && ok) {
    int lo = 0, hi = p.batch;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (static_cast<long long>(s_prefix[mid]) * Hkv <= x) lo = mid; else hi = mid;
    }
    const int seq = lo;
    const int nt = s_prefix[seq + 1] - s_prefix[seq];
    const long long seg_start_seq = static_cast<long long>(s_prefix[seq]) * Hkv;
    const long long rem = x - seg_start_seq;
    const int h = static_cast<int>(rem / nt);
    const int t0 = static_cast<int>(rem - static_cast<long long>(h) * nt);
    const long long seg_start = x - t0;
    const long long seg_end = seg_start + nt;
    const long long my_end = seg_end < r_end ? seg_end : r_end;
    const int t1 = t0 + static_cast<int>(my_end - x);
    int len = p.context_lens[seq];
    len = len > max_len ? max_len : len;

    // query fragments: rows = the G heads sharing kv head h
    uint32_t qa[8][4];
    {
      const __nv_bfloat16* qb = p.q + seq * p.q_row_stride + static_cast<long long>(h) * G * 128;
      const uint32_t* q0 = reinterpret_cast<const uint32_t*>(qb + row * 128);
      const uint32_t* q1 = reinterpret_cast<const uint32_t*>(qb + (row + 8) * 128);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qa[ks][0] = row0_ok ? __ldg(q0 + ks * 8 + quad) : 0u;
        qa[ks][1] = row1_ok ? __ldg(q1 + ks * 8 + quad) : 0u;
        qa[ks][2] = row0_ok ? __ldg(q0 + ks * 8 + 4 + quad) : 0u;
        qa[ks][3] = row1_ok ? __ldg(q1 + ks * 8 + 4 + quad) : 0u;
      }
    }
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int t = t0; t < t1; ++t, ++it) {
      const int stage = it % kDecStages;
      const uint32_t ph = (it / kDecStages) & 1;
      if (!mbar_wait(&bar_full[stage], ph, abort_flag)) { ok = false; break; }
      const int valid = len - (t * kTile + warp * 16);  // valid tokens in this warp's 16-token slab
      if (valid > 0) {
        const uint32_t st = smem_u32(stages + stage * kStageBytes);
        const uint32_t k_base = st, v_base = st + 2 * kSubTileBytes;
        if (valid < 16) {
          // rows past the sequence end hold whatever the cache block holds: zero the V rows so
          // that 0 * garbage cannot produce NaN (K garbage is masked by select below)
          unsigned char* vb = stages + stage * kStageBytes + 2 * kSubTileBytes;
          for (int e = lane; e < 16 * 16; e += 32) {
            const int r = warp * 16 + (e >> 4), c = e & 15;
            if ((e >> 4) >= valid)
              *reinterpret_cast<uint4*>(vb + (c >> 3) * kSubTileBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
                  make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        // ---- S = Q K^T (16 x 16 tokens) ----
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        {
          const int tok = warp * 16 + ((lane >> 4) << 3) + (lane & 7);
          const int dsel = ((lane >> 3) & 1) << 3;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + tile_offset(tok, ks * 16 + dsel, kTile), b0, b1, b2, b3);
            mma_bf16_16816(s[0], qa[ks], b0, b1);
            mma_bf16_16816(s[1], qa[ks], b2, b3);
          }
        }
        // ---- online softmax (log2 domain) ----
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const bool in = (j * 8 + quad * 2 + e) < valid;
            s[j][e] = in ? s[j][e] * p.scale_log2 : -INFINITY;
            s[j][2 + e] = in ? s[j][2 + e] * p.scale_log2 : -INFINITY;
            mx0 = fmaxf(mx0, s[j][e]);
            mx1 = fmaxf(mx1, s[j][2 + e]);
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            s[j][e] = fast_exp2(s[j][e] - mn0);
            s[j][2 + e] = fast_exp2(s[j][2 + e] - mn1);
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
        // ---- O += P V ----
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
        {
          const int tok = warp * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
          const int dsel = (lane >> 4) << 3;
#pragma unroll
          for (int n2 = 0; n2 < 8; ++n2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_base + tile_offset(tok, n2 * 16 + dsel, kTile), b0, b1, b2, b3);
            mma_bf16_16816(o[2 * n2], pa, b0, b1);
            mma_bf16_16816(o[2 * n2 + 1], pa, b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_empty[stage]);
    }
    if (!ok) break;

    // ---- combine the four warps, then either finish the (sequence, head) or leave a partial ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    {
      float* mo = merge_o + warp * G * 128;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        if (row0_ok) *reinterpret_cast<float2*>(mo + row * 128 + n * 8 + quad * 2) = make_float2(o[n][0], o[n][1]);
        if (row1_ok) *reinterpret_cast<float2*>(mo + (row + 8) * 128 + n * 8 + quad * 2) = make_float2(o[n][2], o[n][3]);
      }
      if (quad == 0) {
        float* ml = merge_ml + warp * G * 2;
        if (row0_ok) { ml[row * 2] = m0; ml[row * 2 + 1] = l0; }
        if (row1_ok) { ml[(row + 8) * 2] = m1; ml[(row + 8) * 2 + 1] = l1; }
      }
    }
    named_bar_sync(1, kDecConsumers);
    const bool full = (x == seg_start) && (my_end == seg_end);
    const int slot = static_cast<int>(cta) * 2 + (seg_start <= r_begin ? 0 : 1);
    for (int g = 0; g < G; ++g) {
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < kDecConsumerWarps; ++w) M = fmaxf(M, merge_ml[(w * G + g) * 2]);
      float L = 0.f, acc = 0.f;
#pragma unroll
      for (int w = 0; w < kDecConsumerWarps; ++w) {
        const float wgt = fast_exp2(merge_ml[(w * G + g) * 2] - M);
        L += merge_ml[(w * G + g) * 2 + 1] * wgt;
        acc += merge_o[(w * G + g) * 128 + tid] * wgt;
      }
      if (full) {
        p.out[(static_cast<long long>(seq) * p.H + h * G + g) * 128 + tid] = __float2bfloat16(acc / L);
      } else {
        p.ws_o[(static_cast<long long>(slot) * G + g) * 128 + tid] = acc;
        if (tid == 0) {
          p.ws_ml[(slot * G + g) * 2] = M;
          p.ws_ml[(slot * G + g) * 2 + 1] = L;
        }
      }
    }
    if (!full) {
      // last-arriver merge across the CTAs that share this (sequence, head)
      const long long c_first = ((seg_start + 1) * grid_eff - 1) / T;
      const long long c_last = (seg_end * grid_eff - 1) / T;
      __threadfence();
      named_bar_sync(1, kDecConsumers);
      if (tid == 0) {
        const int old = atomicAdd(&p.counters[seq * Hkv + h], 1);
        s_last = (old == static_cast<int>(c_last - c_first));
      }
      named_bar_sync(1, kDecConsumers);
      if (s_last) {
        __threadfence();
        for (int g = 0; g < G; ++g) {
          float M = -INFINITY, L = 0.f, acc = 0.f;
          for (long long c = c_first; c <= c_last; ++c) {
            const long long cb = c * T / grid_eff;
            const int sl = static_cast<int>(c) * 2 + (seg_start <= cb ? 0 : 1);
            const float2 ml = ld_cg_f32x2(p.ws_ml + (sl * G + g) * 2);
            const float ov = ld_cg_f32(p.ws_o + (static_cast<long long>(sl) * G + g) * 128 + tid);
            const float Mn = fmaxf(M, ml.x);
            const float wa = fast_exp2(M - Mn), wb = fast_exp2(ml.x - Mn);
            L = L * wa + ml.y * wb;
            acc = acc * wa + ov * wb;
            M = Mn;
          }
          p.out[(static_cast<long long>(seq) * p.H + h * G + g) * 128 + tid] = __float2bfloat16(acc / L);
        }
        if (tid == 0) p.counters[seq * Hkv + h] = 0;
      }
    }
    named_bar_sync(1, kDecConsumers);  // merge buffers are reused by the next segment
    x = my_end;
  }
  if (!ok && lane == 0) atomicExch(&g_status_decode, 1);
}

int read_status_decode() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_status_decode, sizeof(int));
  return v;
}

static size_t decode_smem_bytes(int G) {
  return 1024 + static_cast<size_t>(kDecStages) * kStageBytes + static_cast<size_t>(kDecConsumerWarps) * G * 130 * 4 +
         (kDecMaxBatch + 1) * 4 + 64;
}

static int decode_grid() { return 2 * sm_count(); }

static long long decode_partial_bytes(int grid) { return static_cast<long long>(grid) * 2 * kMaxG * 130 * 4; }

}  // namespace b200

extern "C" int64_t b200_decode_workspace_bytes(int32_t max_batch, int32_t num_heads, int32_t num_kv_heads,
                                               int32_t head_dim) {
  using namespace b200;
  if (max_batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || head_dim != 128)
    return set_error(kErrBadShape, "decode_workspace_bytes: bad geometry (batch=%d H=%d Hkv=%d D=%d)", max_batch,
                     num_heads, num_kv_heads, head_dim);
  const int grid = decode_grid();
  if (grid <= 0) return set_error(kErrNoDriver, "decode_workspace_bytes: no CUDA device");
  const long long per_launch = max_batch < kDecMaxBatch ? max_batch : kDecMaxBatch;
  return kWsStatusBytes + decode_partial_bytes(grid) + per_launch * num_kv_heads * 4;
}

extern "C" int b200_decode_attn(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                int64_t num_blocks, int32_t block_size, const int32_t* block_tables,
                                int64_t bt_row_stride, int32_t bt_cols, const int32_t* context_lens, void* out,
                                void* workspace, int64_t workspace_bytes, int32_t batch, int32_t num_heads,
                                int32_t num_kv_heads, int32_t head_dim, float scale, void* stream) {
  using namespace b200;
  if (batch < 0) return set_error(kErrBadShape, "decode_attn: negative batch");
  if (batch == 0) return kOk;
  if (!q || !k_cache || !v_cache || !block_tables || !context_lens || !out)
    return set_error(kErrNullPointer, "decode_attn: null pointer argument");
  if (head_dim != 128) return set_error(kErrBadShape, "decode_attn: head_dim must be 128 (got %d)", head_dim);
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads)
    return set_error(kErrBadShape, "decode_attn: num_heads (%d) must be a positive multiple of num_kv_heads (%d)",
                     num_heads, num_kv_heads);
  const int G = num_heads / num_kv_heads;
  if (G > kMaxG) return set_error(kErrBadShape, "decode_attn: at most %d query heads per kv head (got %d)", kMaxG, G);
  if (block_size <= 0 || block_size % 256)
    return set_error(kErrBadShape, "decode_attn: block_size must be a positive multiple of 256 (got %d)", block_size);
  if (num_blocks <= 0 || num_blocks * block_size >= (1LL << 31))
    return set_error(kErrBadShape, "decode_attn: num_blocks * block_size must be in (0, 2^31)");
  if (bt_cols <= 0 || bt_row_stride < bt_cols || static_cast<long long>(bt_cols) * block_size >= (1LL << 30))
    return set_error(kErrBadShape, "decode_attn: bad block table geometry (cols=%d stride=%lld)", bt_cols,
                     (long long)bt_row_stride);
  if (q_row_stride < static_cast<long long>(num_heads) * 128 || q_row_stride % 8)
    return set_error(kErrMisaligned, "decode_attn: q_row_stride must be >= H*128 and a multiple of 8 elements");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return set_error(kErrMisaligned, "decode_attn: q, caches and out must be 16-byte aligned");
  const int grid = decode_grid();
  if (grid <= 0) return set_error(kErrNoDriver, "decode_attn: no CUDA device");
  const long long per_launch = batch < kDecMaxBatch ? batch : kDecMaxBatch;
  const long long need = kWsStatusBytes + decode_partial_bytes(grid) + per_launch * num_kv_heads * 4;
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return set_error(kErrWorkspace, "decode_attn: workspace of %lld bytes (16-byte aligned, zero-filled once) required, got %lld",
                     need, (long long)workspace_bytes);

  CUtensorMap map_k, map_v;
  int rc = make_tokens_heads_map(&map_k, k_cache, static_cast<uint64_t>(num_blocks) * block_size, num_kv_heads,
                                 static_cast<uint64_t>(num_kv_heads) * 128, kTile);
  if (rc) return rc;
  rc = make_tokens_heads_map(&map_v, v_cache, static_cast<uint64_t>(num_blocks) * block_size, num_kv_heads,
                             static_cast<uint64_t>(num_kv_heads) * 128, kTile);
  if (rc) return rc;

  const size_t smem = decode_smem_bytes(G);
  static std::atomic<size_t> configured{0};
  if (configured.load() < smem) {
    rc = check_cuda(cudaFuncSetAttribute(decode_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem),
                    "decode_attn: cudaFuncSetAttribute");
    if (rc) return rc;
    configured.store(smem);
  }

  unsigned char* ws = static_cast<unsigned char*>(workspace);
  DecodeParams p;
  p.bt_row_stride = bt_row_stride;
  p.bt_cols = bt_cols;
  p.H = num_heads;
  p.Hkv = num_kv_heads;
  p.G = G;
  p.block_size = block_size;
  p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.ws_o = reinterpret_cast<float*>(ws + kWsStatusBytes);
  p.ws_ml = p.ws_o + static_cast<long long>(grid) * 2 * kMaxG * 128;
  p.counters = reinterpret_cast<int*>(ws + kWsStatusBytes + decode_partial_bytes(grid));
  p.q_row_stride = q_row_stride;
  for (int b0 = 0; b0 < batch; b0 += kDecMaxBatch) {
    p.batch = batch - b0 < kDecMaxBatch ? batch - b0 : kDecMaxBatch;
    p.q = static_cast<const __nv_bfloat16*>(q) + b0 * q_row_stride;
    p.out = static_cast<__nv_bfloat16*>(out) + static_cast<long long>(b0) * num_heads * 128;
    p.context_lens = context_lens + b0;
    p.block_tables = block_tables + b0 * bt_row_stride;
    decode_attn_kernel<<<grid, kDecThreads, smem, static_cast<cudaStream_t>(stream)>>>(p, map_k, map_v);
    g_launches.fetch_add(1);
    rc = check_cuda(cudaGetLastError(), "decode_attn launch");
    if (rc) return rc;
  }
  return kOk;
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library have nowhere to get a workspace from: a serving engine that has
// already handed every free byte of the GPU to its KV cache (nano-vllm sizes the cache from the
// free memory it finds, so a later cudaMalloc can fail), a plugin slot whose contract forbids
// allocation inside the call, or code that runs where the framework's caching allocator must not
// be touched.  For them the scratch of the decode kernel lives in the library image itself: a
// file-scope __device__ array that every GPU loading the library holds until the process exits.
// ---------------------------------------------------------------------------------------------
namespace b200 {

constexpr int kStaticMaxGrid = 320;        // persistent CTAs the static scratch has partial slots for
constexpr int kStaticMaxCounters = 8192;   // (sequence, kv head) pairs per launch: min(batch, 1024) * Hkv
constexpr long long kStaticScratchBytes =
    kWsStatusBytes + static_cast<long long>(kStaticMaxGrid) * 2 * kMaxG * 130 * 4 + kStaticMaxCounters * 4;

static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// Device address of the array above on the current device.  In host code the array's name is only a
// handle for the runtime, never an address a kernel may be given, so the address is asked for
// once per device (with that device current) and remembered.
static int static_scratch_address(void** out) {
  static void* cached[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "decode_attn_static: cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return set_error(kErrDevice, "decode_attn_static: device ordinal %d not supported", dev);
  if (!ready[dev].load(std::memory_order_acquire)) {
    void* ptr = nullptr;
    rc = check_cuda(cudaGetSymbolAddress(&ptr, g_decode_static_scratch), "decode_attn_static: cudaGetSymbolAddress");
    if (rc) return rc;
    if (!ptr) return set_error(kErrDevice, "decode_attn_static: the scratch array has no address on device %d", dev);
    cached[dev] = ptr;
    ready[dev].store(1, std::memory_order_release);
  }
  *out = cached[dev];
  return kOk;
}

}  // namespace b200

extern "C" int64_t b200_decode_static_scratch_bytes(void) { return b200::kStaticScratchBytes; }

extern "C" int b200_decode_attn_static(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                       int64_t num_blocks, int32_t block_size, const int32_t* block_tables,
                                       int64_t bt_row_stride, int32_t bt_cols, const int32_t* context_lens, void* out,
                                       int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                       float scale, void* stream) {
  using namespace b200;
  if (batch < 0) return set_error(kErrBadShape, "decode_attn_static: negative batch");
  if (batch == 0) return kOk;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads)
    return set_error(kErrBadShape, "decode_attn_static: num_heads (%d) must be a positive multiple of num_kv_heads (%d)",
                     num_heads, num_kv_heads);
  const int grid = decode_grid();
  if (grid <= 0) return set_error(kErrNoDriver, "decode_attn_static: no CUDA device");
  if (grid > kStaticMaxGrid)
    return set_error(kErrWorkspace,
                     "decode_attn_static: this GPU runs %d persistent CTAs but the built-in scratch has room for %d; "
                     "use b200_decode_attn with a caller-owned workspace", grid, kStaticMaxGrid);
  const long long per_launch = batch < kDecMaxBatch ? batch : kDecMaxBatch;
  if (per_launch * num_kv_heads > kStaticMaxCounters)
    return set_error(kErrWorkspace,
                     "decode_attn_static: min(batch, %d) * num_kv_heads = %lld exceeds the built-in scratch's limit of %d; "
                     "use b200_decode_attn with a caller-owned workspace", kDecMaxBatch, per_launch * num_kv_heads,
                     kStaticMaxCounters);
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  // The array keeps whatever the previous call left.  Partials are always written before they are
  // read; the arrival counters are the one part that must start at zero, so clear them here.
  unsigned char* counters = static_cast<unsigned char*>(scratch) + kWsStatusBytes + decode_partial_bytes(grid);
  rc = check_cuda(cudaMemsetAsync(counters, 0, static_cast<size_t>(per_launch) * num_kv_heads * 4,
                                  static_cast<cudaStream_t>(stream)),
                  "decode_attn_static: clearing the arrival counters");
  if (rc) return rc;
  return b200_decode_attn(q, q_row_stride, k_cache, v_cache, num_blocks, block_size, block_tables, bt_row_stride, bt_cols,
                          context_lens, out, scratch, kStaticScratchBytes, batch, num_heads, num_kv_heads, head_dim,
                          scale, stream);
}
