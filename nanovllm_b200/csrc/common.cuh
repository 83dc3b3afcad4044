// Shared device/host helpers for the paged-KV attention kernels (sm_100a only).
//
// Device side: thin wrappers over the PTX this library is built on -- mbarrier,
// cp.async.bulk.tensor (TMA, never with cluster multicast), ldmatrix, mma.sync -- plus the
// 128-byte-swizzle address arithmetic shared by every tile loader.
// Host side: error recording for the C ABI and CUtensorMap construction through the driver
// entry point obtained at run time (the library does not link libcuda, so it also loads on a
// machine without a GPU driver).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---------------------------------------------------------------------------------------------
// Status codes of the C ABI (negative: rejected before launch; positive: CUDA runtime error)
// ---------------------------------------------------------------------------------------------
enum Status : int {
  kOk = 0,
  kErrNullPointer = -1,
  kErrBadShape = -2,       // unsupported head_dim, H % Hkv, block_size, sizes out of range
  kErrMisaligned = -3,     // pointer or stride not 16-byte aligned
  kErrWorkspace = -4,      // workspace missing or too small
  kErrNoDriver = -5,       // no CUDA driver / device / cuTensorMapEncodeTiled entry point
  kErrTensorMap = -6,      // cuTensorMapEncodeTiled rejected the geometry
  kErrDevice = -7,         // device is not sm_100
  kErrTimeout = -8,        // a bounded device-side wait gave up (reported through the status word)
};

int set_error(int code, const char* fmt, ...);   // records a message, returns code
int check_cuda(cudaError_t e, const char* what); // 0 or positive cudaError_t with message
int sm_count();                                  // multiprocessors of the current device (cached per device)

// Builds a tiled tensor map over a (tokens, heads, 128) bf16 array whose token rows are
// `row_stride_elems` apart: dims {128 head_dim, head, token}, box {64, box_heads, box_tokens}
// (one 64-wide half of head_dim; rows of the box ordered token-major, head-minor), 128-byte
// swizzle.  The same form covers the paged cache (tokens = num_blocks * block_size) and packed
// q/k/v activations with arbitrary row stride.
int make_tokens_heads_map(CUtensorMap* map, const void* base, uint64_t tokens, uint32_t heads,
                          uint64_t row_stride_elems, uint32_t box_tokens, uint32_t box_heads = 1);
int make_tokens_heads_map_cols32(CUtensorMap* map, const void* base, uint64_t tokens, uint32_t heads,
                                 uint64_t row_stride_elems, uint32_t box_tokens, uint32_t box_heads);

#ifdef __CUDACC__

// ---------------------------------------------------------------------------------------------
// Bounded waiting.  Every spin in this library gives up after kSpinLimitCycles (about a second)
// and reports through a status word instead of hanging the GPU.
// ---------------------------------------------------------------------------------------------
constexpr long long kSpinLimitCycles = 2000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Returns false if the wait gave up (caller must unwind; *abort_flag is set for the other roles).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  int spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255) == 0) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kSpinLimitCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// TMA tile load, 3-D, into this CTA's shared memory; completion is signalled on `bar`.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
// TMA tile store, 3-D, from this CTA's shared memory (bulk-group completion).
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Returns once the bulk stores of this thread have finished READING their shared-memory source.
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// The same, but the most recent store may still be reading.
__device__ __forceinline__ void tma_store_wait_read_but_one() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
// Hint: bring one box of a 3-D tensor map into L2 (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Tile layout in shared memory.  A (tokens x 128) bf16 tile is held as two sub-tiles of 64
// columns (128 bytes per row), each written by one TMA box with 128-byte swizzle: the 16-byte
// chunk c of row r sits at chunk (c ^ (r & 7)).  Sub-tile bases are 1024-byte aligned.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t tile_offset(int row, int col /* element, 0..127 */, int rows_per_subtile) {
  const int sub = col >> 6;
  const int chunk = (col & 63) >> 3;
  return static_cast<uint32_t>(sub * rows_per_subtile * 128 + row * 128 + ((chunk ^ (row & 7)) << 4) +
                               ((col & 7) << 1));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8, fp32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Blackwell-only arithmetic used by the softmax loops: 3-input max and packed 2 x fp32 FMA / ADD.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ unsigned long long f32x2_pack(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f32x2_unpack(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long f32x2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long f32x2_add(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ float ld_cg_f32(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ float2 ld_cg_f32x2(const float* p) {
  float2 v;
  asm volatile("ld.global.cg.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "l"(p));
  return v;
}

#endif  // __CUDACC__

}  // namespace b200
