// One launch that puts a decode step's metadata into the static buffers a captured CUDA graph reads.
//
// The reference's model runner prepares a decode step with five host tensors, five host-to-device
// copies (nanovllm/engine/model_runner.py:163-179, :119-123) and then seven device operations that
// move them into the buffers its graphs were captured on (:193-203).  Here the host writes one packed
// record into pinned memory, one copy brings it to the device, and this kernel scatters it:
//   words [0, 2 bs)                 input_ids   int64[bs]
//   words [2 bs, 4 bs)              positions   int64[bs]
//   words [4 bs, 5 bs)              slot_mapping int32[bs]
//   words [5 bs, 6 bs)              context_lens int32[bs]
//   words [6 bs, 6 bs + bs * w)     block_tables int32[bs][w], rows padded with -1
// with exactly the reference's effect on the graph buffers: rows [0, bs) of input_ids and positions
// are written; slot_mapping is -1 and context_lens 0 on every row from bs up to the buffers' length;
// block_tables gets columns [0, w) of rows [0, bs) and keeps whatever else it held (stale tails are
// never dereferenced by the attention kernels).
#include "../../include/b200_attn.h"
#include "kernels.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kMetaThreads = 256;

__global__ void __launch_bounds__(kMetaThreads)
unpack_decode_metadata_kernel(const int* __restrict__ packed, int bs, int w, int rows, int bt_cols,
                              long long* __restrict__ input_ids, long long* __restrict__ positions,
                              int* __restrict__ slot_mapping, int* __restrict__ context_lens,
                              int* __restrict__ block_tables) {
  // (No early trigger of dependent launches here: the decode kernel reads context_lens and the block
  // table ahead of its own dependency wait, which is only sound if whatever writes them has completed.)
  const int tid = blockIdx.x * kMetaThreads + threadIdx.x;
  const int stride = gridDim.x * kMetaThreads;
  const long long* p_ids = reinterpret_cast<const long long*>(packed);
  const long long* p_pos = p_ids + bs;
  const int* p_slot = packed + 4 * bs;
  const int* p_len = p_slot + bs;
  const int* p_bt = p_len + bs;
  for (int i = tid; i < rows; i += stride) {
    const bool live = i < bs;
    if (live) {
      input_ids[i] = p_ids[i];
      positions[i] = p_pos[i];
    }
    slot_mapping[i] = live ? p_slot[i] : -1;
    context_lens[i] = live ? p_len[i] : 0;
  }
  for (int e = tid; e < bs * w; e += stride) {
    const int r = e / w, c = e - r * w;
    block_tables[static_cast<long long>(r) * bt_cols + c] = p_bt[e];
  }
}

}  // namespace b200

extern "C" int b200_unpack_decode_metadata(const void* packed, int32_t batch, int32_t table_width, int32_t buffer_rows,
                                           int32_t buffer_table_cols, int64_t* input_ids, int64_t* positions,
                                           int32_t* slot_mapping, int32_t* context_lens, int32_t* block_tables,
                                           void* stream) {
  using namespace b200;
  if (batch < 0 || table_width < 0 || buffer_rows < 0 || buffer_table_cols < 0)
    return set_error(kErrBadShape, "unpack_decode_metadata: negative size");
  if (batch > buffer_rows || table_width > buffer_table_cols)
    return set_error(kErrBadShape, "unpack_decode_metadata: batch %d x width %d does not fit buffers of %d rows x %d columns",
                     batch, table_width, buffer_rows, buffer_table_cols);
  if (buffer_rows == 0) return kOk;
  if (!packed || !input_ids || !positions || !slot_mapping || !context_lens || !block_tables)
    return set_error(kErrNullPointer, "unpack_decode_metadata: null pointer argument");
  if ((reinterpret_cast<uintptr_t>(packed) | reinterpret_cast<uintptr_t>(input_ids) | reinterpret_cast<uintptr_t>(positions)) & 7)
    return set_error(kErrMisaligned, "unpack_decode_metadata: packed record, input_ids and positions must be 8-byte aligned");
  const long long work = static_cast<long long>(batch) * table_width > buffer_rows ? static_cast<long long>(batch) * table_width
                                                                                   : buffer_rows;
  long long blocks = (work + kMetaThreads - 1) / kMetaThreads;
  if (blocks > 64) blocks = 64;
  unpack_decode_metadata_kernel<<<static_cast<unsigned>(blocks), kMetaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int*>(packed), batch, table_width, buffer_rows, buffer_table_cols,
      reinterpret_cast<long long*>(input_ids), reinterpret_cast<long long*>(positions), slot_mapping, context_lens,
      block_tables);
  g_launches.fetch_add(1);
  return check_cuda(cudaGetLastError(), "unpack_decode_metadata launch");
}
