// store_kvcache: scatter of the step's new K and V rows into the paged cache through
// slot_mapping.  Replaces the reference's Triton kernel (nanovllm/layers/attention.py:10-40).
//
// HBM-bound byte copy: every thread moves 16-byte vectors, consecutive threads take consecutive
// vectors of one row (fully coalesced 128-byte lines on both sides), four independent vectors
// are in flight per thread, offsets are 64-bit, and the grid is a multiple of the SM count.
#include <atomic>

#include "../../include/b200_attn.h"
#include "common.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kStoreThreads = 256;
constexpr int kStoreUnroll = 4;

__global__ void __launch_bounds__(kStoreThreads)
store_kvcache_kernel(const char* __restrict__ key, const char* __restrict__ value, long long key_stride_b,
                     long long value_stride_b, char* __restrict__ k_cache, char* __restrict__ v_cache,
                     const int* __restrict__ slot_mapping, long long total_vecs, int row_vecs, long long n_slots) {
  // Let a dependent launch (the decode kernel that follows in the stream) start its prologue
  // now; it still waits for this grid to finish before it reads the cache.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const long long row_bytes = static_cast<long long>(row_vecs) * 16;
  const long long step = static_cast<long long>(gridDim.x) * kStoreThreads * kStoreUnroll;
  for (long long base = static_cast<long long>(blockIdx.x) * kStoreThreads * kStoreUnroll + threadIdx.x;
       base < total_vecs; base += step) {
    uint4 data[kStoreUnroll];
    char* dst[kStoreUnroll];
#pragma unroll
    for (int u = 0; u < kStoreUnroll; ++u) {
      const long long idx = base + static_cast<long long>(u) * kStoreThreads;
      dst[u] = nullptr;
      if (idx < total_vecs) {
        const long long row = idx / row_vecs;           // (token, K|V) pair
        const int vec = static_cast<int>(idx - row * row_vecs);
        const long long tok = row >> 1;
        const bool is_v = (row & 1) != 0;
        const long long slot = slot_mapping[tok];
        if (slot >= 0 && slot < n_slots) {
          const char* src = (is_v ? value + tok * value_stride_b : key + tok * key_stride_b) + vec * 16;
          data[u] = __ldg(reinterpret_cast<const uint4*>(src));
          dst[u] = (is_v ? v_cache : k_cache) + slot * row_bytes + vec * 16;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kStoreUnroll; ++u)
      if (dst[u]) *reinterpret_cast<uint4*>(dst[u]) = data[u];
  }
}

}  // namespace b200

extern "C" int b200_store_kvcache(const void* key, const void* value, int64_t key_row_stride,
                                  int64_t value_row_stride, void* k_cache, void* v_cache,
                                  const int32_t* slot_mapping, int32_t n_tokens, int32_t row_elems,
                                  int32_t elem_bytes, int64_t n_slots, void* stream) {
  using namespace b200;
  if (n_tokens < 0 || row_elems <= 0 || elem_bytes <= 0 || n_slots < 0 || key_row_stride < 0 || value_row_stride < 0)
    return set_error(kErrBadShape, "store_kvcache: negative or zero size (n_tokens=%d row_elems=%d elem_bytes=%d)",
                     n_tokens, row_elems, elem_bytes);
  if (n_tokens == 0) return kOk;
  if (!key || !value || !k_cache || !v_cache || !slot_mapping)
    return set_error(kErrNullPointer, "store_kvcache: null pointer argument");
  const long long row_bytes = static_cast<long long>(row_elems) * elem_bytes;
  const long long ks = key_row_stride * elem_bytes, vs = value_row_stride * elem_bytes;
  if (row_bytes % 16 || ks % 16 || vs % 16)
    return set_error(kErrMisaligned, "store_kvcache: row bytes (%lld) and row strides (%lld, %lld bytes) must be multiples of 16",
                     row_bytes, ks, vs);
  if ((reinterpret_cast<uintptr_t>(key) | reinterpret_cast<uintptr_t>(value) | reinterpret_cast<uintptr_t>(k_cache) |
       reinterpret_cast<uintptr_t>(v_cache)) & 15)
    return set_error(kErrMisaligned, "store_kvcache: pointers must be 16-byte aligned");
  if (ks < row_bytes || vs < row_bytes)
    return set_error(kErrBadShape, "store_kvcache: row stride smaller than the row");
  const int row_vecs = static_cast<int>(row_bytes / 16);
  const long long total = 2LL * n_tokens * row_vecs;
  const long long per_block = static_cast<long long>(kStoreThreads) * kStoreUnroll;
  long long blocks = (total + per_block - 1) / per_block;
  const int sms = sm_count();
  if (sms <= 0) return set_error(kErrNoDriver, "store_kvcache: no CUDA device");
  const long long cap = static_cast<long long>(sms) * 16;
  if (blocks > cap) blocks = cap;
  store_kvcache_kernel<<<static_cast<unsigned>(blocks), kStoreThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const char*>(key), static_cast<const char*>(value), ks, vs, static_cast<char*>(k_cache),
      static_cast<char*>(v_cache), slot_mapping, total, row_vecs, n_slots);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "store_kvcache launch");
}
