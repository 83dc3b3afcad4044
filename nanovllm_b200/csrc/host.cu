// Host-side plumbing of the C ABI: error strings, device queries, tensor-map construction.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "../../include/b200_attn.h"
#include "kernels.cuh"

namespace b200 {

static thread_local char g_err[512] = "";
std::atomic<long long> g_launches{0};

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return kOk;
  return set_error(static_cast<int>(e), "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

int sm_count() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device attribute: `cache` holds, per device
// ordinal, the largest size already set for `kernel` there.
int ensure_dynamic_smem(const void* kernel, size_t bytes, std::atomic<size_t>* cache, const char* what) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return set_error(kErrDevice, "%s: device ordinal outside [0, %d)", what, kMaxDevices);
  if (cache[dev].load(std::memory_order_acquire) >= bytes) return kOk;
  const int rc = check_cuda(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)), what);
  if (rc) return rc;
  cache[dev].store(bytes, std::memory_order_release);
  return kOk;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static std::once_flag once;
  static EncodeTiledFn fn = nullptr;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
    cudaGetLastError();
  });
  return fn;
}

int make_tokens_heads_map(CUtensorMap* map, const void* base, uint64_t tokens, uint32_t heads,
                          uint64_t row_stride_elems, uint32_t box_tokens, uint32_t box_heads) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(kErrNoDriver, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  if (tokens == 0) tokens = 1;  // an empty tensor is never read; keep the encoder happy
  cuuint64_t dims[3] = {128, heads, tokens};
  cuuint64_t strides[2] = {128 * 2, row_stride_elems * 2};
  cuuint32_t box[3] = {64, box_heads, box_tokens};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(kErrTensorMap, "cuTensorMapEncodeTiled failed with CUresult %d (tokens=%llu heads=%u stride=%llu)",
                     static_cast<int>(r), (unsigned long long)tokens, heads, (unsigned long long)row_stride_elems);
  return kOk;
}

// Output form of the same map: boxes of {32 dims, box_heads, box_tokens} with a 64-byte swizzle
// (a box row is 64 bytes; 16-byte chunk c of row r sits at chunk c ^ ((r >> 1) & 3)).
int make_tokens_heads_map_cols32(CUtensorMap* map, const void* base, uint64_t tokens, uint32_t heads,
                                 uint64_t row_stride_elems, uint32_t box_tokens, uint32_t box_heads) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(kErrNoDriver, "cuTensorMapEncodeTiled is not available (no CUDA driver?)");
  if (tokens == 0) tokens = 1;
  cuuint64_t dims[3] = {128, heads, tokens};
  cuuint64_t strides[2] = {128 * 2, row_stride_elems * 2};
  cuuint32_t box[3] = {32, box_heads, box_tokens};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(kErrTensorMap, "cuTensorMapEncodeTiled (output map) failed with CUresult %d (tokens=%llu heads=%u)",
                     static_cast<int>(r), (unsigned long long)tokens, heads);
  return kOk;
}

}  // namespace b200

extern "C" {

int b200_version(void) { return B200_ATTN_VERSION; }

const char* b200_last_error(void) { return b200::g_err; }

int64_t b200_launch_count(void) { return b200::g_launches.load(); }

int b200_device_status(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) {
    cudaError_t e = cudaGetLastError();
    return b200::check_cuda(e == cudaSuccess ? cudaErrorUnknown : e, "device_status: cudaDeviceSynchronize");
  }
  const int sd = b200::read_status_decode(), sm = b200::read_status_prefill_mma(), st = b200::read_status_prefill_tc2();
  if (sd || sm || st) {
    // Report once and recover: clear the status words and the library's own launch-to-launch state, so that the
    // next call of this function speaks about later launches only and the next prefill starts from ticket 0.
    int rc = b200::reset_state_decode();
    if (!rc) rc = b200::reset_state_prefill_mma();
    if (!rc) rc = b200::reset_state_prefill_tc2();
    if (rc) return rc;
    return b200::set_error(b200::kErrTimeout,
                           "a bounded device-side wait gave up (decode=%d prefill mma.sync=%d prefill tcgen05=%d); the "
                           "library's own state has been reset, a decode workspace used by the failed call must be "
                           "zero-filled again by its owner",
                           sd, sm, st);
  }
  return b200::kOk;
}

int b200_test_inject_timeout(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return b200::check_cuda(cudaGetLastError(), "test_inject_timeout: cudaDeviceSynchronize");
  return b200::inject_timeout_prefill_tc2();
}

}  // extern "C"
