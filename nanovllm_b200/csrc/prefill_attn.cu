// C-ABI entry point of prefill attention: argument checks, tensor maps, kernel selection.
#include "../../include/b200_attn.h"
#include "kernels.cuh"

extern "C" int b200_prefill_attn(const void* q, int64_t q_row_stride, const void* k, const void* v,
                                 int64_t k_row_stride, int64_t v_row_stride, int64_t total_k, const void* k_cache,
                                 const void* v_cache, int64_t num_blocks, int32_t block_size,
                                 const int32_t* block_tables, int64_t bt_row_stride, int32_t bt_cols,
                                 const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, int32_t batch,
                                 int32_t total_q, int32_t max_seqlen_q, int32_t max_seqlen_k, void* out,
                                 int32_t num_heads, int32_t num_kv_heads, int32_t head_dim, float scale,
                                 int32_t kernel_variant, void* stream) {
  using namespace b200;
  if (batch < 0 || total_q < 0) return set_error(kErrBadShape, "prefill_attn: negative batch or total_q");
  if (batch == 0 || total_q == 0) return kOk;
  if (!q || !out || !cu_seqlens_q || !cu_seqlens_k) return set_error(kErrNullPointer, "prefill_attn: null pointer argument");
  if (head_dim != 128) return set_error(kErrBadShape, "prefill_attn: head_dim must be 128 (got %d)", head_dim);
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads)
    return set_error(kErrBadShape, "prefill_attn: num_heads (%d) must be a positive multiple of num_kv_heads (%d)",
                     num_heads, num_kv_heads);
  const int G = num_heads / num_kv_heads;
  if (G > 128) return set_error(kErrBadShape, "prefill_attn: at most 128 query heads per kv head");
  if (q_row_stride < static_cast<long long>(num_heads) * 128 || q_row_stride % 8)
    return set_error(kErrMisaligned, "prefill_attn: q_row_stride must be >= H*128 and a multiple of 8 elements");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15)
    return set_error(kErrMisaligned, "prefill_attn: q and out must be 16-byte aligned");
  if (max_seqlen_q <= 0 || max_seqlen_k <= 0)
    return set_error(kErrBadShape, "prefill_attn: max_seqlen_q/k must be positive");

  if (kernel_variant < 0 || kernel_variant > 2)
    return set_error(kErrBadShape, "prefill_attn: kernel_variant must be 0 .. 2");
  const bool tc_ok = 128 % G == 0;
  if (kernel_variant == 2 && !tc_ok)
    return set_error(kErrBadShape, "prefill_attn: the tcgen05 kernel needs 128 %% (num_heads / num_kv_heads) == 0 (got %d)", G);
  const bool use_tc = kernel_variant == 2 || (kernel_variant == 0 && tc_ok);
  const uint32_t kv_box = use_tc ? 128 : 64;
  CUtensorMap map_k, map_v;
  const bool paged = block_tables != nullptr;
  int rc;
  if (paged) {
    if (!k_cache || !v_cache) return set_error(kErrNullPointer, "prefill_attn: block_tables given without caches");
    if (block_size <= 0 || block_size % 256)
      return set_error(kErrBadShape, "prefill_attn: block_size must be a positive multiple of 256 (got %d)", block_size);
    if (num_blocks <= 0 || num_blocks * block_size >= (1LL << 31))
      return set_error(kErrBadShape, "prefill_attn: num_blocks * block_size must be in (0, 2^31)");
    if (bt_cols <= 0 || bt_row_stride < bt_cols)
      return set_error(kErrBadShape, "prefill_attn: bad block table geometry");
    if ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15)
      return set_error(kErrMisaligned, "prefill_attn: caches must be 16-byte aligned");
    const uint64_t rows = static_cast<uint64_t>(num_blocks) * block_size;
    rc = make_tokens_heads_map(&map_k, k_cache, rows, num_kv_heads, static_cast<uint64_t>(num_kv_heads) * 128, kv_box);
    if (rc) return rc;
    rc = make_tokens_heads_map(&map_v, v_cache, rows, num_kv_heads, static_cast<uint64_t>(num_kv_heads) * 128, kv_box);
    if (rc) return rc;
  } else {
    if (!k || !v) return set_error(kErrNullPointer, "prefill_attn: dense k/v missing");
    if (total_k <= 0 || total_k >= (1LL << 31)) return set_error(kErrBadShape, "prefill_attn: total_k out of range");
    if (k_row_stride < static_cast<long long>(num_kv_heads) * 128 || v_row_stride < static_cast<long long>(num_kv_heads) * 128 ||
        k_row_stride % 8 || v_row_stride % 8)
      return set_error(kErrMisaligned, "prefill_attn: k/v row strides must be >= Hkv*128 and multiples of 8 elements");
    if ((reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v)) & 15)
      return set_error(kErrMisaligned, "prefill_attn: k and v must be 16-byte aligned");
    rc = make_tokens_heads_map(&map_k, k, static_cast<uint64_t>(total_k), num_kv_heads, static_cast<uint64_t>(k_row_stride), kv_box);
    if (rc) return rc;
    rc = make_tokens_heads_map(&map_v, v, static_cast<uint64_t>(total_k), num_kv_heads, static_cast<uint64_t>(v_row_stride), kv_box);
    if (rc) return rc;
  }

  PrefillParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_row_stride = q_row_stride;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.cu_q = cu_seqlens_q;
  p.cu_k = cu_seqlens_k;
  p.block_tables = block_tables;
  p.bt_row_stride = bt_row_stride;
  p.bt_cols = bt_cols;
  p.block_size = paged ? block_size : 256;
  p.num_blocks = num_blocks;
  p.batch = batch;
  p.H = num_heads;
  p.Hkv = num_kv_heads;
  p.G = G;
  p.QT = 128 / G;
  p.n_slots = total_q / p.QT + batch;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.total_q = total_q;
  p.max_seqlen_q = max_seqlen_q;
  p.max_seqlen_k = max_seqlen_k;
  p.out_tma = 0;
  if (use_tc) {
    CUtensorMap map_q;
    rc = make_tokens_heads_map(&map_q, q, static_cast<uint64_t>(total_q), num_heads, static_cast<uint64_t>(q_row_stride),
                               static_cast<uint32_t>(p.QT), static_cast<uint32_t>(G));
    if (rc) return rc;
    // output map of the persistent kernel: boxes of 32 tile rows = (32 / G tokens) x (G heads) x 32 dims
    CUtensorMap map_o = map_q;
    p.out_tma = 32 % G == 0;
    if (p.out_tma) {
      rc = make_tokens_heads_map_cols32(&map_o, out, static_cast<uint64_t>(total_q), num_heads,
                                        static_cast<uint64_t>(num_heads) * 128, static_cast<uint32_t>(32 / G),
                                        static_cast<uint32_t>(G));
      if (rc) return rc;
    }
    return launch_prefill_tc2(p, map_q, map_k, map_v, map_o, static_cast<cudaStream_t>(stream));
  }
  return launch_prefill_mma(p, map_k, map_v, static_cast<cudaStream_t>(stream));
}
