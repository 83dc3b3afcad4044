// Declarations shared between the translation units of the library: prefill parameters and
// launchers, and the per-unit device status words.
#pragma once
#include "common.cuh"

namespace b200 {

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
// tcgen05 variant: Q map with a {64, G, 128 / G} box, K/V maps with 128-token boxes; needs 128 % G == 0.
bool prefill_tc_supports(const PrefillParams& p);
int launch_prefill_tc(const PrefillParams& p, const CUtensorMap& map_q, const CUtensorMap& map_k,
                      const CUtensorMap& map_v, cudaStream_t stream);

// tcgen05 variant, persistent with two query tiles per CTA sharing each K/V tile (same maps as above).
int launch_prefill_tc2(PrefillParams p, const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                       const CUtensorMap& map_o, cudaStream_t stream);

// tcgen05 variant, persistent, 64-key steps with double-buffered S (K/V maps with 64-token boxes).
int launch_prefill_tc3(PrefillParams p, const CUtensorMap& map_q, const CUtensorMap& map_k, const CUtensorMap& map_v,
                       cudaStream_t stream);

// Device-side "a bounded wait gave up" flags, one per translation unit, summed by b200_device_status().
int read_status_decode();
int read_status_prefill_mma();
int read_status_prefill_tc();
int read_status_prefill_tc2();
int read_status_prefill_tc3();

}  // namespace b200
