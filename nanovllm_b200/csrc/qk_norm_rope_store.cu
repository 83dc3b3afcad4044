// Producer side of the attention layer in one launch: per-head RMSNorm of q and k, rotary
// embedding, and the store of k and v into the paged cache.  Replaces, for one decoder layer,
//   q_norm / k_norm      nanovllm/layers/layernorm.py:16-26    (called at nanovllm/models/qwen3.py:76-77)
//   rotary_emb           nanovllm/layers/rotary_embedding.py:6-14, 37-48  (called at models/qwen3.py:79)
//   store_kvcache        nanovllm/layers/attention.py:10-40    (called at layers/attention.py:62-63)
// which the reference runs as three compiled element-wise kernels plus one Triton kernel.
//
// A half-warp owns one 128-element head vector of one token: lane j of 16 holds elements [8j, 8j + 8)
// (16-byte accesses), so the rotary partner (element i +- 64) of every element sits in lane j ^ 8.  q heads and k heads are
// normalised in fp32, cast to bf16, multiplied by the bf16 weight, rotated in fp32 (products and
// sums rounded separately, as the reference's eager arithmetic does) and written out contiguous;
// k is also written to its cache slot.  v heads are copied bit-for-bit from the strided qkv row to
// their cache slot.  Pure streaming: HBM / launch bound, no tensor-core work.
#include <atomic>

#include <cuda_bf16.h>

#include "../../include/b200_attn.h"
#include "common.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

struct QkNormRopeParams {
  const __nv_bfloat16* qkv;
  long long qkv_row_stride;            // elements
  const long long* positions;          // (n_tokens) int64
  const __nv_bfloat16* q_weight;       // (128)
  const __nv_bfloat16* k_weight;       // (128)
  const float* cos_sin;                // (max_position, 128): 64 cos then 64 sin
  int max_position;
  float eps;
  __nv_bfloat16* q_out;                // (n_tokens, H, 128)
  __nv_bfloat16* k_out;                // (n_tokens, Hkv, 128)
  __nv_bfloat16* k_cache;              // flat rows of Hkv * 128 elements, or nullptr
  __nv_bfloat16* v_cache;
  const int* slot_mapping;             // (n_tokens) or nullptr
  long long n_slots;
  int n_tokens, H, Hkv;
};

constexpr int kQkThreads = 256;     // 16 head vectors per CTA pass: one per half-warp

__device__ __forceinline__ void bf16x8_to_float(const uint4& r, float (&x)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __low2float(h[i]);
    x[2 * i + 1] = __high2float(h[i]);
  }
}

// One head vector: `raw` holds this lane's 8 elements of head `hd` of token `tok`.
__device__ __forceinline__ void qk_one_vector(const QkNormRopeParams& p, int tok, int hd, const uint4& raw, int sub,
                                              unsigned half_mask) {
  long long slot = -1;
  if (p.slot_mapping && p.k_cache && p.v_cache) {
    slot = p.slot_mapping[tok];
    if (slot >= p.n_slots) slot = -1;                    // never write outside the cache
  }
  if (hd >= p.H + p.Hkv) {
    // v head: a bit copy into the cache
    if (slot >= 0)
      *reinterpret_cast<uint4*>(p.v_cache + (slot * p.Hkv + (hd - p.H - p.Hkv)) * 128 + sub * 8) = raw;
    return;
  }
  const bool is_q = hd < p.H;
  long long pos = p.positions[tok];
  pos = pos < 0 ? 0 : (pos >= p.max_position ? p.max_position - 1 : pos);
  const float* cs = p.cos_sin + pos * 128 + (sub & 7) * 8;
  const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(cs + 64), s1 = *reinterpret_cast<const float4*>(cs + 68);
  const uint4 wraw = *reinterpret_cast<const uint4*>((is_q ? p.q_weight : p.k_weight) + sub * 8);
  float x[8], w[8];
  bf16x8_to_float(raw, x);
  bf16x8_to_float(wraw, w);
  // mean of squares over the 128 elements, fp32
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = __fadd_rn(ss, __fmul_rn(x[i], x[i]));
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(half_mask, ss, o);
  const float rinv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.f), p.eps));
  const float cosv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
  const float sinv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
  // normalise in fp32, round to bf16, scale by the bf16 weight (rounded to bf16 again); the results are
  // exact bf16 values, so they travel to the partner lane as packed pairs (4 shuffles instead of 8)
  uint32_t ap[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __nv_bfloat162 n2 = __floats2bfloat162_rn(__fmul_rn(x[2 * i], rinv), __fmul_rn(x[2 * i + 1], rinv));
    ap[i] = pack_bf16(__fmul_rn(__low2float(n2), w[2 * i]), __fmul_rn(__high2float(n2), w[2 * i + 1]));
  }
  float y[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t bp = __shfl_xor_sync(half_mask, ap[i], 8);       // the elements 64 away
    const __nv_bfloat162 a2 = *reinterpret_cast<const __nv_bfloat162*>(&ap[i]);
    const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&bp);
    const float a0 = __low2float(a2), a1 = __high2float(a2), b0 = __low2float(b2), b1 = __high2float(b2);
    // first half:  y1 = x1 * cos - x2 * sin      second half:  y2 = x2 * cos + x1 * sin
    const float t0 = __fmul_rn(b0, sinv[2 * i]), t1 = __fmul_rn(b1, sinv[2 * i + 1]);
    y[2 * i] = __fadd_rn(__fmul_rn(a0, cosv[2 * i]), sub < 8 ? -t0 : t0);
    y[2 * i + 1] = __fadd_rn(__fmul_rn(a1, cosv[2 * i + 1]), sub < 8 ? -t1 : t1);
  }
  uint4 outw;
  outw.x = pack_bf16(y[0], y[1]);
  outw.y = pack_bf16(y[2], y[3]);
  outw.z = pack_bf16(y[4], y[5]);
  outw.w = pack_bf16(y[6], y[7]);
  if (is_q) {
    *reinterpret_cast<uint4*>(p.q_out + (static_cast<long long>(tok) * p.H + hd) * 128 + sub * 8) = outw;
  } else {
    const int kh = hd - p.H;
    *reinterpret_cast<uint4*>(p.k_out + (static_cast<long long>(tok) * p.Hkv + kh) * 128 + sub * 8) = outw;
    if (slot >= 0) *reinterpret_cast<uint4*>(p.k_cache + (slot * p.Hkv + kh) * 128 + sub * 8) = outw;
  }
}

__global__ void __launch_bounds__(kQkThreads, 4)
qk_norm_rope_store_kernel(const QkNormRopeParams p) {
  // a half-warp owns one head vector: lane j of 16 holds elements [8j, 8j + 8) (one 16-byte access),
  // the rotary partner (element i +- 64) of each of them sits in lane j ^ 8; two vectors are in flight
  // per half-warp so that the second load is on its way while the first is worked on
  const int sub = threadIdx.x & 15;
  const int heads = p.H + 2 * p.Hkv;
  const long long n_vec = static_cast<long long>(p.n_tokens) * heads;
  const long long stride = static_cast<long long>(gridDim.x) * (kQkThreads / 16);
  const unsigned half_mask = 0xffffu << (threadIdx.x & 16);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (long long vec = static_cast<long long>(blockIdx.x) * (kQkThreads / 16) + (threadIdx.x >> 4); vec < n_vec;
       vec += 2 * stride) {
    const long long vec2 = vec + stride;
    const int tok = static_cast<int>(vec / heads);
    const int hd = static_cast<int>(vec - static_cast<long long>(tok) * heads);
    const bool two = vec2 < n_vec;
    const int tok2 = two ? static_cast<int>(vec2 / heads) : tok;
    const int hd2 = two ? static_cast<int>(vec2 - static_cast<long long>(tok2) * heads) : hd;
    const uint4 raw = *reinterpret_cast<const uint4*>(p.qkv + tok * p.qkv_row_stride + hd * 128 + sub * 8);
    const uint4 raw2 = *reinterpret_cast<const uint4*>(p.qkv + tok2 * p.qkv_row_stride + hd2 * 128 + sub * 8);
    qk_one_vector(p, tok, hd, raw, sub, half_mask);
    if (two) qk_one_vector(p, tok2, hd2, raw2, sub, half_mask);
  }
}

}  // namespace b200

extern "C" int b200_qk_norm_rope_store(const void* qkv, int64_t qkv_row_stride, const int64_t* positions,
                                       const void* q_weight, const void* k_weight, const float* cos_sin_cache,
                                       int32_t max_position, float eps, void* q_out, void* k_out, void* k_cache,
                                       void* v_cache, const int32_t* slot_mapping, int64_t n_slots, int32_t n_tokens,
                                       int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, void* stream) {
  using namespace b200;
  if (n_tokens == 0) return kOk;
  if (!qkv || !positions || !q_weight || !k_weight || !cos_sin_cache || !q_out || !k_out)
    return set_error(kErrNullPointer, "qk_norm_rope_store: null pointer");
  if (head_dim != 128 || num_heads <= 0 || num_kv_heads <= 0 || n_tokens < 0 || max_position <= 0)
    return set_error(kErrBadShape, "qk_norm_rope_store: head_dim must be 128 and the counts positive (H=%d Hkv=%d D=%d n=%d)",
                     num_heads, num_kv_heads, head_dim, n_tokens);
  if ((k_cache == nullptr) != (v_cache == nullptr))
    return set_error(kErrNullPointer, "qk_norm_rope_store: k_cache and v_cache must both be given or both be null");
  if (k_cache && !slot_mapping) return set_error(kErrNullPointer, "qk_norm_rope_store: a cache needs slot_mapping");
  if (k_cache && n_slots <= 0) return set_error(kErrBadShape, "qk_norm_rope_store: n_slots must be positive");
  const long long width = static_cast<long long>(num_heads + 2 * num_kv_heads) * 128;
  if (qkv_row_stride < width || qkv_row_stride % 8 != 0)
    return set_error(kErrMisaligned, "qk_norm_rope_store: qkv_row_stride must be >= (H + 2 Hkv) * 128 and a multiple of 8 elements");
  auto mis = [](const void* ptr, uintptr_t a) { return ptr && (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) != 0; };
  if (mis(qkv, 16) || mis(q_out, 16) || mis(k_out, 16) || mis(k_cache, 16) || mis(v_cache, 16) || mis(q_weight, 16) ||
      mis(k_weight, 16) || mis(cos_sin_cache, 16))
    return set_error(kErrMisaligned, "qk_norm_rope_store: every tensor must be 16-byte aligned");
  QkNormRopeParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.qkv_row_stride = qkv_row_stride;
  p.positions = reinterpret_cast<const long long*>(positions);
  p.q_weight = static_cast<const __nv_bfloat16*>(q_weight);
  p.k_weight = static_cast<const __nv_bfloat16*>(k_weight);
  p.cos_sin = cos_sin_cache;
  p.max_position = max_position;
  p.eps = eps;
  p.q_out = static_cast<__nv_bfloat16*>(q_out);
  p.k_out = static_cast<__nv_bfloat16*>(k_out);
  p.k_cache = static_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = static_cast<__nv_bfloat16*>(v_cache);
  p.slot_mapping = slot_mapping;
  p.n_slots = n_slots;
  p.n_tokens = n_tokens;
  p.H = num_heads;
  p.Hkv = num_kv_heads;
  const long long n_vec = static_cast<long long>(n_tokens) * (num_heads + 2 * num_kv_heads);
  const int sms = sm_count();
  if (sms <= 0) return set_error(kErrNoDriver, "qk_norm_rope_store: no CUDA device");
  const long long want = (n_vec + kQkThreads / 16 - 1) / (kQkThreads / 16);
  const int grid = static_cast<int>(want < static_cast<long long>(sms) * 8 ? want : static_cast<long long>(sms) * 8);
  qk_norm_rope_store_kernel<<<grid, kQkThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "qk_norm_rope_store launch");
}
