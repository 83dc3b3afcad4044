// One-shot all-reduce (sum) of a small bf16 message across the tensor-parallel ranks of one node,
// over plain peer loads and stores (CUDA IPC mappings of every rank's exchange buffer; no multimem,
// no TMA, no library kernel on peer memory).  Replaces, for decode-sized messages, the NCCL call
// after the row-parallel output projection (nanovllm/layers/linear.py:149-153, `dist.all_reduce(y)`):
// 56 of them per decode step of a 28-layer model, each at most batch x hidden x 2 bytes (512 KiB at
// batch 256, hidden 1024), where a ring or tree collective is pure latency.
//
// Every rank owns an exchange buffer that all ranks have mapped:
//   data   two slots of kArMaxBytes (calls alternate, so a rank that is already in the next call never
//          overwrites what a slower rank is still reading)
//   flags  [kArMaxCtas][kArMaxRanks] epoch words, written by the peers, polled locally
// CTA c of every rank handles slice c of the message, and only ever waits for CTA c of the other
// ranks: (A) copy the slice of the input into the own data slot, (B) store the call's epoch into the
// flag word (c, own rank) of EVERY rank (release at system scope after a CTA barrier), (C) wait until
// the own flag words (c, r) of all ranks r have reached the epoch (acquire loads of LOCAL memory;
// bounded: after the limit the CTA records a status and leaves its slice unwritten), (D) load the
// slice from every rank's slot and add in fp32 in rank order -- the same order on every rank, so all
// ranks end up with identical bits -- and write bf16 back in place.
// The epoch of a CTA index lives in local device memory and is advanced by the kernel itself, so a
// captured launch can be replayed; all ranks must issue the same sequence of calls (same sizes).
#include <cstring>

#include "../../include/b200_attn.h"
#include "kernels.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kArMaxRanks = 8;
constexpr int kArMaxCtas = 64;
constexpr int kArThreads = 512;
constexpr long long kArMaxBytes = 512 * 1024;           // per message
constexpr long long kArDataBytes = 2 * kArMaxBytes;     // two slots
constexpr long long kArFlagBytes = kArMaxCtas * kArMaxRanks * 4;

struct ArParams {
  unsigned char* peer[kArMaxRanks];     // every rank's exchange buffer as mapped here (own included)
  unsigned int* epochs;                 // [kArMaxCtas] local
  int* status;                          // local: set to 1 if a wait gave up
  __nv_bfloat16* inout;
  long long n_elems;
  long long chunk_elems;                // per CTA, a multiple of 8
  long long spin_limit;                 // cycles
  int rank, world;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kArThreads)
small_allreduce_kernel(const ArParams p) {
  __shared__ unsigned int s_epoch;
  __shared__ int s_fail;
  const int c = blockIdx.x, tid = threadIdx.x;
  if (tid == 0) {
    s_epoch = p.epochs[c] + 1;
    s_fail = 0;
  }
  __syncthreads();
  const unsigned int e = s_epoch;
  const long long slot_off = static_cast<long long>(e & 1u) * kArMaxBytes;
  const long long begin = static_cast<long long>(c) * p.chunk_elems;
  long long end = begin + p.chunk_elems;
  if (end > p.n_elems) end = p.n_elems;
  const long long nvec = begin < end ? (end - begin + 7) / 8 : 0;      // 16-byte vectors (n_elems is a multiple of 8)
  // (A) the slice of the input into this rank's slot
  {
    const uint4* src = reinterpret_cast<const uint4*>(p.inout + begin);
    uint4* dst = reinterpret_cast<uint4*>(p.peer[p.rank] + slot_off + begin * 2);
    for (long long v = tid; v < nvec; v += kArThreads) dst[v] = src[v];
  }
  __syncthreads();
  // (B) tell every rank (this one included) that slice c of this rank is in place
  if (tid < p.world) {
    __threadfence_system();
    unsigned int* flags = reinterpret_cast<unsigned int*>(p.peer[tid] + kArDataBytes);
    st_release_sys(flags + c * kArMaxRanks + p.rank, e);
  }
  // (C) wait for slice c of every rank
  if (tid < p.world) {
    const unsigned int* mine = reinterpret_cast<const unsigned int*>(p.peer[p.rank] + kArDataBytes) + c * kArMaxRanks + tid;
    const long long t0 = clock64();
    int spins = 0;
    // epochs only grow; a peer may already have signalled the next call
    while (static_cast<int>(ld_acquire_sys(mine) - e) < 0) {
      if ((++spins & 63) == 0 && clock64() - t0 > p.spin_limit) {
        s_fail = 1;
        break;
      }
    }
  }
  __syncthreads();
  if (s_fail) {
    if (tid == 0) {
      atomicExch(p.status, 1);
      p.epochs[c] = e;
    }
    return;
  }
  // (D) sum in rank order, fp32, one rounding
  uint4* out = reinterpret_cast<uint4*>(p.inout + begin);
  for (long long v = tid; v < nvec; v += kArThreads) {
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    uint4 raw[kArMaxRanks];
#pragma unroll
    for (int r = 0; r < kArMaxRanks; ++r)
      if (r < p.world) raw[r] = ld_volatile_v4(p.peer[r] + slot_off + begin * 2 + v * 16);
#pragma unroll
    for (int r = 0; r < kArMaxRanks; ++r) {
      if (r < p.world) {
        const uint32_t w[4] = {raw[r].x, raw[r].y, raw[r].z, raw[r].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          acc[2 * i] += __uint_as_float(w[i] << 16);
          acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
        }
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    out[v] = o;
  }
  if (tid == 0) p.epochs[c] = e;
}

}  // namespace b200

extern "C" int64_t b200_small_allreduce_buffer_bytes(void) { return b200::kArDataBytes + b200::kArFlagBytes; }
extern "C" int64_t b200_small_allreduce_state_bytes(void) { return b200::kArMaxCtas * 4 + 64; }
extern "C" int64_t b200_small_allreduce_max_bytes(void) { return b200::kArMaxBytes; }

extern "C" int b200_small_allreduce(void* const* peer_buffers, int32_t rank, int32_t world, void* local_state,
                                    void* inout, int64_t n_elems, double wait_limit_seconds, void* stream) {
  using namespace b200;
  if (world < 1 || world > kArMaxRanks || rank < 0 || rank >= world)
    return set_error(kErrBadShape, "small_allreduce: rank %d of %d (at most %d ranks)", rank, world, kArMaxRanks);
  if (n_elems < 0 || n_elems % 8) return set_error(kErrBadShape, "small_allreduce: n_elems must be a non-negative multiple of 8");
  if (n_elems * 2 > kArMaxBytes)
    return set_error(kErrBadShape, "small_allreduce: %lld bytes exceed the %lld-byte message limit", (long long)(n_elems * 2),
                     (long long)kArMaxBytes);
  if (n_elems == 0) return kOk;
  if (!peer_buffers || !local_state || !inout) return set_error(kErrNullPointer, "small_allreduce: null pointer argument");
  if (reinterpret_cast<uintptr_t>(inout) & 15) return set_error(kErrMisaligned, "small_allreduce: the message must be 16-byte aligned");
  ArParams p;
  for (int r = 0; r < kArMaxRanks; ++r) {
    p.peer[r] = r < world ? static_cast<unsigned char*>(peer_buffers[r]) : nullptr;
    if (r < world && (!p.peer[r] || (reinterpret_cast<uintptr_t>(p.peer[r]) & 15)))
      return set_error(kErrNullPointer, "small_allreduce: exchange buffer of rank %d missing or misaligned", r);
  }
  p.epochs = static_cast<unsigned int*>(local_state);
  p.status = reinterpret_cast<int*>(static_cast<unsigned char*>(local_state) + kArMaxCtas * 4);
  p.inout = static_cast<__nv_bfloat16*>(inout);
  p.n_elems = n_elems;
  p.rank = rank;
  p.world = world;
  // 16 KiB of the message per CTA, at most kArMaxCtas of them; the same on every rank for the same size
  long long ctas = (n_elems * 2 + 16383) / 16384;
  if (ctas > kArMaxCtas) ctas = kArMaxCtas;
  long long chunk = (n_elems + ctas - 1) / ctas;
  chunk = (chunk + 7) / 8 * 8;
  p.chunk_elems = chunk;
  ctas = (n_elems + chunk - 1) / chunk;
  if (wait_limit_seconds <= 0.0 || wait_limit_seconds > 10.0) wait_limit_seconds = 1.0;
  p.spin_limit = static_cast<long long>(wait_limit_seconds * 2.0e9);
  small_allreduce_kernel<<<static_cast<unsigned>(ctas), kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "small_allreduce launch");
}

extern "C" int b200_small_allreduce_status(const void* local_state) {
  using namespace b200;
  if (!local_state) return set_error(kErrNullPointer, "small_allreduce_status: null pointer");
  if (cudaDeviceSynchronize() != cudaSuccess)
    return check_cuda(cudaGetLastError(), "small_allreduce_status: cudaDeviceSynchronize");
  int v = 0;
  const int rc = check_cuda(cudaMemcpy(&v, static_cast<const unsigned char*>(local_state) + kArMaxCtas * 4, sizeof(int),
                                       cudaMemcpyDeviceToHost),
                            "small_allreduce_status: reading the status word");
  if (rc) return rc;
  if (v) return set_error(kErrTimeout, "small_allreduce: a rank's peers did not arrive within the wait limit");
  return kOk;
}

// ---- set-up helpers: sharing an exchange buffer between the ranks' processes ------------------------
// cudaIpcGetMemHandle names the whole allocation a pointer lies in; the buffer handed in is usually a piece of a
// larger block of the framework's caching allocator, so the distance from the block's start travels with the handle.
extern "C" int b200_ipc_export(const void* ptr, void* handle_out_64_bytes, int64_t* offset_out) {
  using namespace b200;
  if (!ptr || !handle_out_64_bytes || !offset_out) return set_error(kErrNullPointer, "ipc_export: null pointer argument");
  typedef CUresult (*GetAttrFn)(void*, CUpointer_attribute, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuPointerGetAttribute", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    return set_error(kErrNoDriver, "ipc_export: cuPointerGetAttribute is not available");
  }
  CUdeviceptr base = 0;
  const CUresult r = reinterpret_cast<GetAttrFn>(fn)(&base, CU_POINTER_ATTRIBUTE_RANGE_START_ADDR, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS || !base) return set_error(kErrDevice, "ipc_export: cannot find the allocation of %p (CUresult %d)", ptr, (int)r);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  const int rc = check_cuda(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle_out_64_bytes), reinterpret_cast<void*>(base)),
                            "ipc_export: cudaIpcGetMemHandle (memory from an expandable-segments allocator cannot be shared this way)");
  if (rc) return rc;
  *offset_out = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return kOk;
}

// Maps another process's exported buffer into the current device's address space (peer access is enabled by the
// runtime when the buffer lives on another GPU).  The mapping stays until the process exits.
extern "C" int b200_ipc_open(const void* handle_64_bytes, int64_t offset, void** ptr_out) {
  using namespace b200;
  if (!handle_64_bytes || !ptr_out || offset < 0) return set_error(kErrNullPointer, "ipc_open: bad argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64_bytes, sizeof(h));
  void* base = nullptr;
  const int rc = check_cuda(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess), "ipc_open: cudaIpcOpenMemHandle");
  if (rc) return rc;
  *ptr_out = static_cast<unsigned char*>(base) + offset;
  return kOk;
}
