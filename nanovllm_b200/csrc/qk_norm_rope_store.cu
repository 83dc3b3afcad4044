// Producer side of the attention layer in one launch: per-head RMSNorm of q and k, rotary
// embedding, and the store of k and v into the paged cache.  Replaces, for one decoder layer,
//   q_norm / k_norm      nanovllm/layers/layernorm.py:16-26    (called at nanovllm/models/qwen3.py:76-77)
//   rotary_emb           nanovllm/layers/rotary_embedding.py:6-14, 37-48  (called at models/qwen3.py:79)
//   store_kvcache        nanovllm/layers/attention.py:10-40    (called at layers/attention.py:62-63)
// which the reference runs as three compiled element-wise kernels plus one Triton kernel.
//
// A half-warp owns one 128-element head vector at a time (four consecutive heads of a token per pass):
// lane j of 16 holds elements [8j, 8j + 8)
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

constexpr int kQkThreads = 256;     // 16 half-warps per CTA
constexpr int kQkGroup = 4;         // head vectors of one token a half-warp works through per pass (large batches)

__device__ __forceinline__ unsigned long long f32x2_mul(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// bf16 pair -> packed fp32 pair (exact)
__device__ __forceinline__ unsigned long long bf16x2_to_f32x2(uint32_t v) {
  return f32x2_pack(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}

// What a half-warp needs once per token (not once per head): where the token goes in the cache and this
// lane's eight cos / sin values of its position.
struct QkTokenCtx {
  long long slot;                      // -1: no store
  unsigned long long cosv[4], sinv[4]; // packed pairs; sin carries the sign of this lane's half (-sin for the first)
};

__device__ __forceinline__ QkTokenCtx qk_token_ctx(const QkNormRopeParams& p, int tok, int sub) {
  QkTokenCtx c;
  c.slot = -1;
  if (p.slot_mapping && p.k_cache && p.v_cache) {
    c.slot = p.slot_mapping[tok];
    if (c.slot >= p.n_slots) c.slot = -1;                // never write outside the cache
  }
  long long pos = p.positions[tok];
  pos = pos < 0 ? 0 : (pos >= p.max_position ? p.max_position - 1 : pos);
  const float* cs = p.cos_sin + pos * 128 + (sub & 7) * 8;
  const float4 c0 = *reinterpret_cast<const float4*>(cs), c1 = *reinterpret_cast<const float4*>(cs + 4);
  const float4 s0 = *reinterpret_cast<const float4*>(cs + 64), s1 = *reinterpret_cast<const float4*>(cs + 68);
  // first half:  y1 = x1 * cos - x2 * sin      second half:  y2 = x2 * cos + x1 * sin
  // (negating sin is exact, and a + (-t) rounds like a - t)
  const float sg = sub < 8 ? -1.f : 1.f;
  c.cosv[0] = f32x2_pack(c0.x, c0.y); c.cosv[1] = f32x2_pack(c0.z, c0.w);
  c.cosv[2] = f32x2_pack(c1.x, c1.y); c.cosv[3] = f32x2_pack(c1.z, c1.w);
  c.sinv[0] = f32x2_pack(sg * s0.x, sg * s0.y); c.sinv[1] = f32x2_pack(sg * s0.z, sg * s0.w);
  c.sinv[2] = f32x2_pack(sg * s1.x, sg * s1.y); c.sinv[3] = f32x2_pack(sg * s1.z, sg * s1.w);
  return c;
}

// One q or k head vector: `raw` holds this lane's 8 elements; `w` the lane's 8 weights as packed fp32 pairs.
// Every product and every sum is rounded on its own (mul.rn / add.rn, packed two at a time), in the order the
// reference's eager arithmetic takes them.
__device__ __forceinline__ uint4 qk_norm_rope_vector(const uint4& raw, const unsigned long long (&w)[4],
                                                     const QkTokenCtx& c, float eps, unsigned half_mask) {
  const uint32_t r[4] = {raw.x, raw.y, raw.z, raw.w};
  unsigned long long x[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) x[i] = bf16x2_to_f32x2(r[i]);
  // mean of squares over the 128 elements, fp32
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float q0, q1;
    f32x2_unpack(f32x2_mul(x[i], x[i]), q0, q1);
    ss = __fadd_rn(__fadd_rn(ss, q0), q1);
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(half_mask, ss, o);
  const float rinv = __frsqrt_rn(__fadd_rn(__fdiv_rn(ss, 128.f), eps));
  const unsigned long long rinv2 = f32x2_pack(rinv, rinv);
  // normalise in fp32, round to bf16, scale by the bf16 weight (rounded to bf16 again); the results are
  // exact bf16 values, so they travel to the partner lane as packed pairs (4 shuffles instead of 8)
  uint32_t ap[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float n0, n1, m0, m1;
    f32x2_unpack(f32x2_mul(x[i], rinv2), n0, n1);
    f32x2_unpack(f32x2_mul(bf16x2_to_f32x2(pack_bf16(n0, n1)), w[i]), m0, m1);
    ap[i] = pack_bf16(m0, m1);
  }
  uint32_t y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t bp = __shfl_xor_sync(half_mask, ap[i], 8);       // the elements 64 away
    float y0, y1;
    f32x2_unpack(f32x2_add(f32x2_mul(bf16x2_to_f32x2(ap[i]), c.cosv[i]), f32x2_mul(bf16x2_to_f32x2(bp), c.sinv[i])), y0, y1);
    y[i] = pack_bf16(y0, y1);
  }
  return make_uint4(y[0], y[1], y[2], y[3]);
}

__device__ __forceinline__ void qk_weight_pairs(const __nv_bfloat16* wt, int sub, unsigned long long (&w)[4]) {
  const uint4 wraw = *reinterpret_cast<const uint4*>(wt + sub * 8);
  w[0] = bf16x2_to_f32x2(wraw.x); w[1] = bf16x2_to_f32x2(wraw.y);
  w[2] = bf16x2_to_f32x2(wraw.z); w[3] = bf16x2_to_f32x2(wraw.w);
}

template <int GROUP>
__global__ void __launch_bounds__(kQkThreads, GROUP == 1 ? 4 : 3)
qk_norm_rope_store_kernel(const QkNormRopeParams p) {
  // A half-warp owns one head vector at a time: lane j of 16 holds elements [8j, 8j + 8) (one 16-byte access),
  // the rotary partner (element i +- 64) of each of them sits in lane j ^ 8.  It takes GROUP consecutive
  // heads of one token per pass -- all loads of the pass go out first -- so that what belongs to the token
  // (slot, position, the lane's cos / sin values) and to the head kind (the norm weight) is fetched once per
  // pass instead of once per head.  GROUP = 1 for decode-sized batches, where the launch is latency bound
  // and more half-warps in flight matter more than the instructions saved.
  const int sub = threadIdx.x & 15;
  const int heads = p.H + 2 * p.Hkv;
  const int groups = (heads + GROUP - 1) / GROUP;                       // per token
  const long long n_units = static_cast<long long>(p.n_tokens) * groups;
  const long long stride = static_cast<long long>(gridDim.x) * (kQkThreads / 16);
  const unsigned half_mask = 0xffffu << (threadIdx.x & 16);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  unsigned long long wq[4], wk[4];
  if (GROUP > 1) {
    qk_weight_pairs(p.q_weight, sub, wq);
    qk_weight_pairs(p.k_weight, sub, wk);
  }
  for (long long unit = static_cast<long long>(blockIdx.x) * (kQkThreads / 16) + (threadIdx.x >> 4); unit < n_units;
       unit += stride) {
    const int tok = static_cast<int>(unit / groups);
    const int hd0 = static_cast<int>(unit - static_cast<long long>(tok) * groups) * GROUP;
    const __nv_bfloat16* row = p.qkv + tok * p.qkv_row_stride + sub * 8;
    uint4 raw[GROUP];
#pragma unroll
    for (int g = 0; g < GROUP; ++g)
      if (hd0 + g < heads) raw[g] = *reinterpret_cast<const uint4*>(row + (hd0 + g) * 128);
    if (GROUP == 1 && hd0 < p.H + p.Hkv) {
      // one head per pass: only the weight of its kind (both sets would cost registers the pass does not have)
      qk_weight_pairs(hd0 < p.H ? p.q_weight : p.k_weight, sub, wq);
#pragma unroll
      for (int i = 0; i < 4; ++i) wk[i] = wq[i];
    }
    const QkTokenCtx c = qk_token_ctx(p, tok, sub);
#pragma unroll
    for (int g = 0; g < GROUP; ++g) {
      const int hd = hd0 + g;
      if (hd >= heads) break;
      if (hd >= p.H + p.Hkv) {
        // v head: a bit copy into the cache
        if (c.slot >= 0)
          *reinterpret_cast<uint4*>(p.v_cache + (c.slot * p.Hkv + (hd - p.H - p.Hkv)) * 128 + sub * 8) = raw[g];
      } else if (hd < p.H) {
        const uint4 outw = qk_norm_rope_vector(raw[g], wq, c, p.eps, half_mask);
        *reinterpret_cast<uint4*>(p.q_out + (static_cast<long long>(tok) * p.H + hd) * 128 + sub * 8) = outw;
      } else {
        const int kh = hd - p.H;
        const uint4 outw = qk_norm_rope_vector(raw[g], wk, c, p.eps, half_mask);
        *reinterpret_cast<uint4*>(p.k_out + (static_cast<long long>(tok) * p.Hkv + kh) * 128 + sub * 8) = outw;
        if (c.slot >= 0) *reinterpret_cast<uint4*>(p.k_cache + (c.slot * p.Hkv + kh) * 128 + sub * 8) = outw;
      }
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
  const int sms = sm_count();
  if (sms <= 0) return set_error(kErrNoDriver, "qk_norm_rope_store: no CUDA device");
  const int heads = num_heads + 2 * num_kv_heads;
  // one head per pass while that still leaves fewer half-warps than the device can hold
  const bool small = static_cast<long long>(n_tokens) * heads <= static_cast<long long>(sms) * 6 * (kQkThreads / 16);
  const int group = small ? 1 : kQkGroup;
  const long long n_units = static_cast<long long>(n_tokens) * ((heads + group - 1) / group);
  const long long want = (n_units + kQkThreads / 16 - 1) / (kQkThreads / 16);
  const long long cap = static_cast<long long>(sms) * (small ? 8 : 6);
  const int grid = static_cast<int>(want < cap ? want : cap);
  if (small)
    qk_norm_rope_store_kernel<1><<<grid, kQkThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    qk_norm_rope_store_kernel<kQkGroup><<<grid, kQkThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "qk_norm_rope_store launch");
}
