// Producer side of the attention layer in one launch: per-head RMSNorm of q and k, rotary
// embedding, and the store of k and v into the paged cache.  Replaces, for one decoder layer,
//   q_norm / k_norm      nanovllm/layers/layernorm.py:16-26    (called at nanovllm/models/qwen3.py:76-77)
//   rotary_emb           nanovllm/layers/rotary_embedding.py:6-14, 37-48  (called at models/qwen3.py:79)
//   store_kvcache        nanovllm/layers/attention.py:10-40    (called at layers/attention.py:62-63)
// which the reference runs as three compiled element-wise kernels plus one Triton kernel.
//
// One warp owns one 128-element head vector of one token: lane l holds elements [4l, 4l + 4), so the
// rotary partner (element i +- 64) of every element sits in lane l ^ 16.  q heads and k heads are
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

constexpr int kQkWarps = 8;

__global__ void __launch_bounds__(kQkWarps * 32)
qk_norm_rope_store_kernel(const QkNormRopeParams p) {
  const int lane = threadIdx.x & 31;
  const int heads = p.H + 2 * p.Hkv;
  const long long n_vec = static_cast<long long>(p.n_tokens) * heads;
  const long long stride = static_cast<long long>(gridDim.x) * kQkWarps;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  for (long long vec = static_cast<long long>(blockIdx.x) * kQkWarps + (threadIdx.x >> 5); vec < n_vec; vec += stride) {
    const int tok = static_cast<int>(vec / heads);
    const int hd = static_cast<int>(vec - static_cast<long long>(tok) * heads);
    const uint2 raw = *reinterpret_cast<const uint2*>(p.qkv + tok * p.qkv_row_stride + hd * 128 + lane * 4);
    long long slot = -1;
    if (p.slot_mapping && p.k_cache && p.v_cache) {
      slot = p.slot_mapping[tok];
      if (slot >= p.n_slots) slot = -1;                    // never write outside the cache
    }
    if (hd >= p.H + p.Hkv) {
      // v head: a bit copy into the cache
      if (slot >= 0)
        *reinterpret_cast<uint2*>(p.v_cache + (slot * p.Hkv + (hd - p.H - p.Hkv)) * 128 + lane * 4) = raw;
      continue;
    }
    const bool is_q = hd < p.H;
    const __nv_bfloat162 r01 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 r23 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    float x[4] = {__low2float(r01), __high2float(r01), __low2float(r23), __high2float(r23)};
    // mean of squares over the 128 elements, fp32
    float ss = __fadd_rn(__fadd_rn(__fmul_rn(x[0], x[0]), __fmul_rn(x[1], x[1])),
                         __fadd_rn(__fmul_rn(x[2], x[2]), __fmul_rn(x[3], x[3])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rinv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.f), p.eps));
    const uint2 wraw = *reinterpret_cast<const uint2*>((is_q ? p.q_weight : p.k_weight) + lane * 4);
    const __nv_bfloat162 w01 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.x);
    const __nv_bfloat162 w23 = *reinterpret_cast<const __nv_bfloat162*>(&wraw.y);
    const float w[4] = {__low2float(w01), __high2float(w01), __low2float(w23), __high2float(w23)};
    long long pos = p.positions[tok];
    pos = pos < 0 ? 0 : (pos >= p.max_position ? p.max_position - 1 : pos);
    const float* cs = p.cos_sin + pos * 128 + (lane & 15) * 4;
    const float4 c4 = *reinterpret_cast<const float4*>(cs);
    const float4 s4 = *reinterpret_cast<const float4*>(cs + 64);
    const float cosv[4] = {c4.x, c4.y, c4.z, c4.w}, sinv[4] = {s4.x, s4.y, s4.z, s4.w};
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      // normalise in fp32, round to bf16, scale by the bf16 weight (rounded to bf16 again)
      const float xn = __bfloat162float(__float2bfloat16_rn(__fmul_rn(x[i], rinv)));
      const float a = __bfloat162float(__float2bfloat16_rn(__fmul_rn(xn, w[i])));
      const float b = __shfl_xor_sync(0xffffffffu, a, 16);          // the element 64 away
      // first half:  y1 = x1 * cos - x2 * sin      second half:  y2 = x2 * cos + x1 * sin
      y[i] = lane < 16 ? __fsub_rn(__fmul_rn(a, cosv[i]), __fmul_rn(b, sinv[i]))
                       : __fadd_rn(__fmul_rn(a, cosv[i]), __fmul_rn(b, sinv[i]));
    }
    uint2 outw;
    outw.x = pack_bf16(y[0], y[1]);
    outw.y = pack_bf16(y[2], y[3]);
    if (is_q) {
      *reinterpret_cast<uint2*>(p.q_out + (static_cast<long long>(tok) * p.H + hd) * 128 + lane * 4) = outw;
    } else {
      const int kh = hd - p.H;
      *reinterpret_cast<uint2*>(p.k_out + (static_cast<long long>(tok) * p.Hkv + kh) * 128 + lane * 4) = outw;
      if (slot >= 0) *reinterpret_cast<uint2*>(p.k_cache + (slot * p.Hkv + kh) * 128 + lane * 4) = outw;
    }
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
  if (qkv_row_stride < width || qkv_row_stride % 4 != 0)
    return set_error(kErrMisaligned, "qk_norm_rope_store: qkv_row_stride must be >= (H + 2 Hkv) * 128 and a multiple of 4 elements");
  auto mis = [](const void* ptr, uintptr_t a) { return ptr && (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) != 0; };
  if (mis(qkv, 8) || mis(q_out, 8) || mis(k_out, 8) || mis(k_cache, 8) || mis(v_cache, 8) || mis(q_weight, 8) ||
      mis(k_weight, 8) || mis(cos_sin_cache, 16))
    return set_error(kErrMisaligned, "qk_norm_rope_store: tensors must be 8-byte aligned (the cos/sin table 16-byte)");
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
  const long long want = (n_vec + kQkWarps - 1) / kQkWarps;
  const int grid = static_cast<int>(want < static_cast<long long>(sms) * 8 ? want : static_cast<long long>(sms) * 8);
  qk_norm_rope_store_kernel<<<grid, kQkWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "qk_norm_rope_store launch");
}
