// Declarations shared between the translation units of the library: prefill parameters and
// launchers, and the per-unit device status words.
#pragma once
#include <atomic>

#include "common.cuh"

namespace b200 {

constexpr int kMaxDevices = 64;   // device ordinals the per-device caches of the host side cover

// Raises the dynamic shared memory limit of `kernel` on the current device if `cache[device]` says it
// has not been raised that far yet (the attribute is per device; `cache` has kMaxDevices entries).
int ensure_dynamic_smem(const void* kernel, size_t bytes, std::atomic<size_t>* cache, const char* what);

struct PrefillParams {
  const __nv_bfloat16* q;
  long long q_row_stride;
  __nv_bfloat16* out;  // (total_q, H, 128) contiguous
  const int* cu_q;
  const int* cu_k;
  const int* block_tables;  // nullptr: dense K/V
  long long bt_row_stride;
  int bt_cols;
  int block_size;
  long long num_blocks;
  int batch, H, Hkv, G, QT;
  int n_slots;  // upper bound on query tiles: total_q / QT + batch
  int total_q, max_seqlen_q, max_seqlen_k;
  float scale_log2;
  int out_tma;  // tc2: the output map (boxes of 32 tile rows) is usable: 32 % G == 0
};

// mma.sync variant: K/V maps with 64-token boxes.
int launch_prefill_mma(const PrefillParams& p, const CUtensorMap& map_k, const CUtensorMap& map_v, cudaStream_t stream);
// tcgen05 variant, persistent with two query tiles per CTA sharing each K/V tile: Q map with a
// {64, G, 128 / G} box, K/V maps with 128-token boxes; needs 128 % G == 0.
int launch_prefill_tc2(PrefillParams p, const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                       const CUtensorMap& map_o, cudaStream_t stream);

// Device-side "a bounded wait gave up" flags, one per translation unit, read by b200_device_status().
// The reset functions clear the flag and whatever launch-to-launch state of the unit an abandoned
// launch may have left behind (the tcgen05 kernel's ticket counter).
int read_status_decode();
int read_status_prefill_mma();
int read_status_prefill_tc2();
int reset_state_decode();
int reset_state_prefill_mma();
int reset_state_prefill_tc2();
int inject_timeout_prefill_tc2();   // test hook: leaves the unit as an abandoned launch would

}  // namespace b200
