// One-shot all-reduce (sum) of a small bf16 message across the tensor-parallel ranks of one node,
// over plain peer stores (CUDA IPC mappings of every rank's exchange buffer; no multimem, no TMA, no
// library kernel on peer memory).  Replaces, for decode-sized messages, the NCCL call after the
// row-parallel output projection (nanovllm/layers/linear.py:149-153, `dist.all_reduce(y)`): 56 of them
// per decode step of a 28-layer model, each at most batch x hidden x 2 bytes (512 KiB at batch 256,
// hidden 1024), where a collective is pure latency.
//
// Push, with the flag travelling inside the data: every rank owns an exchange buffer that all ranks
// have mapped, laid out [2 slots][source rank][message as 16-byte words].  A sender writes each 8 bytes
// of its message (4 bf16) as one 16-byte word {data, epoch, data, epoch} straight into the region that
// is its own in every peer's buffer; a receiver polls its LOCAL buffer word by word until both epoch
// fields of a word equal the call's epoch, and adds the ranks' values in fp32 in rank order (the same
// order everywhere: all ranks end up with identical bits).  No fence, no barrier, no read over NVLink:
// the latency of a call is one posted store across the link plus a local poll.  Calls alternate
// between the two slots, so a rank that is already in the next call never overwrites words a slower
// rank is still waiting for (to get two calls ahead it would need that rank's data of the call in
// between).  The epoch is one word of local device memory, read by every CTA on entry and advanced by
// the last CTA to leave, so a captured launch can be replayed; it is unique per call, which is what
// makes a stale word from any earlier call (of whatever size) impossible to mistake for a fresh one.
// All ranks must issue the same sequence of calls.  Every poll is bounded: after the limit the thread
// records a status and leaves its part of the message unchanged.
#include <cstring>

#include "../../include/b200_attn.h"
#include "kernels.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kArMaxRanks = 8;
constexpr int kArMaxCtas = 32;
constexpr int kArThreads = 512;
constexpr long long kArMaxBytes = 512 * 1024;                       // per message
constexpr long long kArRegionBytes = 2 * kArMaxBytes;               // a message as flagged 16-byte words
constexpr long long kArSlotBytes = kArMaxRanks * kArRegionBytes;    // one region per source rank
constexpr long long kArBufferBytes = 2 * kArSlotBytes;              // two slots
constexpr int kArStateWords = 4;                                    // epoch, CTAs done, status, pad

struct ArParams {
  unsigned char* peer[kArMaxRanks];     // every rank's exchange buffer as mapped here (own included)
  unsigned int* state;                  // local: [0] epoch of the last finished call, [1] CTAs done, [2] status
  __nv_bfloat16* inout;
  long long n_words;                    // 8-byte payload words (4 bf16 each)
  long long spin_limit;                 // cycles
  int rank, world;
};

__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(kArThreads)
small_allreduce_kernel(const ArParams p) {
  __shared__ unsigned int s_epoch;
  const int tid = threadIdx.x;
  if (tid == 0) s_epoch = *reinterpret_cast<volatile unsigned int*>(p.state) + 1;
  __syncthreads();
  const unsigned int e = s_epoch;
  const long long slot_off = static_cast<long long>(e & 1u) * kArSlotBytes;
  const long long stride = static_cast<long long>(gridDim.x) * kArThreads;
  const long long first = static_cast<long long>(blockIdx.x) * kArThreads + tid;
  const uint2* in = reinterpret_cast<const uint2*>(p.inout);
  // push: this rank's words into its region of every peer's buffer
  for (long long w = first; w < p.n_words; w += stride) {
    const uint2 x = in[w];
    const uint4 flagged = make_uint4(x.x, e, x.y, e);
#pragma unroll
    for (int r = 0; r < kArMaxRanks; ++r)
      if (r < p.world && r != p.rank)
        st_volatile_v4(p.peer[r] + slot_off + static_cast<long long>(p.rank) * kArRegionBytes + w * 16, flagged);
  }
  // gather: the peers' words as they land in the local buffer, summed in rank order
  const unsigned char* mine = p.peer[p.rank] + slot_off;
  bool failed = false;
  const long long t0 = clock64();
  uint2* out = reinterpret_cast<uint2*>(p.inout);
  for (long long w = first; w < p.n_words && !failed; w += stride) {
    const uint2 own = in[w];
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < kArMaxRanks; ++r) {
      if (r >= p.world) break;
      uint32_t lo, hi;
      if (r == p.rank) {
        lo = own.x;
        hi = own.y;
      } else {
        const unsigned char* src = mine + static_cast<long long>(r) * kArRegionBytes + w * 16;
        uint4 v = ld_volatile_v4(src);
        int spins = 0;
        while (v.y != e || v.w != e) {
          if ((++spins & 63) == 0 && clock64() - t0 > p.spin_limit) {
            failed = true;
            break;
          }
          v = ld_volatile_v4(src);
        }
        lo = v.x;
        hi = v.z;
      }
      acc[0] += __uint_as_float(lo << 16);
      acc[1] += __uint_as_float(lo & 0xffff0000u);
      acc[2] += __uint_as_float(hi << 16);
      acc[3] += __uint_as_float(hi & 0xffff0000u);
    }
    if (!failed) out[w] = make_uint2(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]));
  }
  if (failed) atomicExch(p.state + 2, 1u);
  // the last CTA to leave advances the epoch (every CTA has read it by then)
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const unsigned int done = atomicAdd(p.state + 1, 1u);
    if (done == gridDim.x - 1) {
      p.state[1] = 0;
      __threadfence();
      *reinterpret_cast<volatile unsigned int*>(p.state) = e;
    }
  }
}

}  // namespace b200

extern "C" int64_t b200_small_allreduce_buffer_bytes(void) { return b200::kArBufferBytes; }
extern "C" int64_t b200_small_allreduce_state_bytes(void) { return b200::kArStateWords * 4; }
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
  p.state = static_cast<unsigned int*>(local_state);
  p.inout = static_cast<__nv_bfloat16*>(inout);
  p.n_words = n_elems / 4;
  p.rank = rank;
  p.world = world;
  // 8 KiB of the message per CTA, at most kArMaxCtas of them; the same on every rank for the same size
  long long ctas = (n_elems * 2 + 8191) / 8192;
  if (ctas > kArMaxCtas) ctas = kArMaxCtas;
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
  const int rc = check_cuda(cudaMemcpy(&v, static_cast<const unsigned char*>(local_state) + 8, sizeof(int),
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
