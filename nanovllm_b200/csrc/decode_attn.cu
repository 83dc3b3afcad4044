// Paged single-token decode attention (replaces flash_attn_with_kvcache as called at
// nanovllm/layers/attention.py:71-74).
//
// HBM-bound: every K and V byte of every context token is read exactly once.  Design:
//  * Work unit = one 64-token tile of one (sequence, kv head).  The tiles of all sequences and
//    heads form one flat list (sequence -> head -> tile), derived on the device from context_lens
//    by a block scan in every CTA: the launch geometry never depends on device data, as CUDA-graph
//    replay requires.  The list is cut into contiguous PIECES: one equal static piece per CTA
//    of the persistent grid (2 CTAs per SM) covering about 70 % of the tiles, then one larger and
//    four smaller pieces per CTA handed out through an atomic ticket counter, so that CTAs that
//    stream faster take more of the tail and all finish together.
//  * The producer warp (one elected lane) walks its pieces.  For every (sequence, head) segment it
//    publishes a descriptor in shared memory, bulk-copies the segment's G query rows into a small
//    ring, and issues the TMA tile loads (two 64x64 boxes for K, two for V, 128-byte swizzle;
//    16-token boxes for the ragged last tile of a sequence) into a ring of stages guarded by
//    full/empty mbarriers.  The descriptor and the query rows ride on the full-barrier of the
//    segment's first tile, and metadata of the next segment is fetched one segment ahead, so the
//    ring never drains at sequence or piece boundaries.
//  * Four consumer warps take 16 tokens of each tile: QK^T and PV on mma.sync.m16n8k16 (the G
//    query heads of the kv head are rows of the 16-row A operand), online softmax in fp32 with
//    quad shuffles.  At the end of a segment they only drop their running (m, l, O) into shared
//    memory and go on with the next tile.
//  * An epilogue warp combines the four warps' states and writes the bf16 row, or, where a piece
//    boundary cuts the (sequence, head), a partial (m, l, unnormalised O) to the workspace; the
//    last piece to arrive (one atomic counter per (sequence, head), reset by that warp) merges the
//    partials.  No CTA ever waits for another; every mbarrier wait is bounded.
#include "../../include/b200_attn.h"
#include "kernels.cuh"

namespace b200 {
extern std::atomic<long long> g_launches;

constexpr int kTile = 64;                       // tokens per stage
constexpr int kSubTileBytes = kTile * 128;      // 64 tokens x 64 dims bf16
constexpr int kStageBytes = 4 * kSubTileBytes;  // K lo, K hi, V lo, V hi
constexpr int kDecStages = 3;
constexpr int kDecConsumerWarps = 4;
constexpr int kDecConsumers = kDecConsumerWarps * 32;
constexpr int kDecProducerWarp = kDecConsumerWarps;
constexpr int kDecEpilogueWarp = kDecConsumerWarps + 1;
constexpr int kDecThreads = kDecConsumers + 64;
constexpr int kDecMaxBatch = 512;               // per launch; the host splits larger batches
constexpr int kDecPer = (kDecMaxBatch + kDecThreads - 1) / kDecThreads;
constexpr int kMaxG = 16;
constexpr int kWsStatusBytes = 256;  // header: word 0 is the ticket counter of the piece scheduler
constexpr int kWsCounterInts = kDecMaxBatch * 128;   // arrival counters: fixed region, up to 128 kv heads
constexpr int kSegRing = kDecStages + 1;   // segment descriptors / query rows in flight
constexpr int kDecPending = 8;             // partials written but not yet counted, per CTA
// Geometry of the dynamic tail of the piece scheduler (measured on B200): used from 256 tiles per CTA;
// one piece of 15 % and four of 3.75 % of a CTA's equal share are handed out through tickets.
constexpr int kDynFactor = 256, kDynBigPct = 15, kDynSmallPct100 = 375, kDynSmallN = 4;
static __device__ int g_status_decode = 0;

struct DecodeParams {
  const __nv_bfloat16* q;
  long long q_row_stride;
  __nv_bfloat16* out;
  const int* context_lens;
  const int* block_tables;
  long long bt_row_stride;
  int bt_cols;
  int batch, H, Hkv, G;
  int block_size;
  long long num_blocks;
  float scale_log2;
  int n_merge;    // hand-off buffers between the consumer warps and the epilogue warp (1 or 2)
  int dyn_factor; // work per CTA (tiles) from which the dynamic tail is used
  int big_pct, small_pct100, small_n;  // geometry of the dynamic tail
  float* ws_o;    // [2 * pieces][G][128] unnormalised partial outputs
  float* ws_ml;   // [2 * pieces][G][2]   running max (log2 domain) and sum
  int* counters;  // [batch * Hkv], zero between launches
  unsigned int* ticket;  // piece scheduler, zero between launches
};


// One (sequence, kv head) segment inside one piece, as the producer hands it to the other warps.
struct SegDesc {
  int seq;               // -1: no more work for this CTA
  int h;
  int t0, t1;            // tiles [t0, t1) of the (sequence, head) that lie in the piece
  int nt;                // tiles of the whole (sequence, head)
  int len;               // context length, clamped to the block table's capacity
  int slot;              // workspace slot for a partial: 2 * piece + (does the piece start inside it ? 0 : 1)
  int pad;
  long long seg_start;   // flat position of tile 0 of the (sequence, head)
};

// How the flat tile list [0, T) is cut into pieces.  Pieces are numbered in list order:
//   [0, g)            static, one per CTA, equal sizes, together the first Ts tiles;
//   [g, g + nb)       "big" dynamic pieces of Cb tiles;
//   [g + nb, total)   "small" dynamic pieces of Cs tiles, ending exactly at T.
// Every CTA computes the same geometry from T and the grid size.
struct DecPieces {
  long long T, Ts, Tb_end;
  int g, nb, ns, Cb, Cs;
  __device__ __forceinline__ int dynamic() const { return nb + ns; }
  __device__ __forceinline__ long long start(int i) const {
    if (i < g) return static_cast<long long>(i) * Ts / g;
    if (i < g + nb) return Ts + static_cast<long long>(i - g) * Cb;
    return Tb_end + static_cast<long long>(i - g - nb) * Cs;
  }
  __device__ __forceinline__ int of(long long x) const {
    if (x < Ts) return static_cast<int>(((x + 1) * g - 1) / Ts);
    if (x < Tb_end) return g + static_cast<int>((x - Ts) / Cb);
    return g + nb + static_cast<int>((x - Tb_end) / Cs);
  }
};

__device__ __forceinline__ DecPieces dec_pieces(long long T, int grid, int dyn_factor, int big_pct, int small_pct100,
                                              int small_n) {
  DecPieces pc;
  pc.T = T;
  pc.g = T < grid ? static_cast<int>(T) : grid;
  if (T < static_cast<long long>(dyn_factor) * grid) {          // too little work to be worth a dynamic tail
    pc.Ts = pc.Tb_end = T;
    pc.nb = pc.ns = 0;
    pc.Cb = pc.Cs = 1;
    return pc;
  }
  const long long W = T / grid;   // tiles per CTA if all ran at the same speed
  pc.Cs = static_cast<int>((W * small_pct100 + 5000) / 10000);   // small_pct100 / 100 % of W each, small_n per CTA
  pc.Cb = static_cast<int>((W * big_pct + 50) / 100);            // big_pct % of W, one per CTA
  if (pc.Cs < 1) pc.Cs = 1;
  if (pc.Cb < 1) pc.Cb = 1;
  pc.nb = grid;
  pc.ns = small_n * grid;
  pc.Ts = T - static_cast<long long>(pc.nb) * pc.Cb - static_cast<long long>(pc.ns) * pc.Cs;
  pc.Tb_end = pc.Ts + static_cast<long long>(pc.nb) * pc.Cb;
  return pc;
}

// The segment that starts at flat position x inside a piece [.., r_end).
__device__ __forceinline__ SegDesc dec_locate(const int* s_prefix, int batch, int Hkv, long long x, long long r_begin,
                                              long long r_end, int piece) {
  int lo = 0, hi = batch;
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (static_cast<long long>(s_prefix[mid]) * Hkv <= x) lo = mid; else hi = mid;
  }
  SegDesc d;
  d.seq = lo;
  d.nt = s_prefix[lo + 1] - s_prefix[lo];
  const long long rem = x - static_cast<long long>(s_prefix[lo]) * Hkv;
  d.h = static_cast<int>(rem / d.nt);
  d.t0 = static_cast<int>(rem - static_cast<long long>(d.h) * d.nt);
  d.seg_start = x - d.t0;
  const long long seg_end = d.seg_start + d.nt;
  const long long my_end = seg_end < r_end ? seg_end : r_end;
  d.t1 = d.t0 + static_cast<int>(my_end - x);
  d.slot = piece * 2 + (d.seg_start <= r_begin ? 0 : 1);
  d.len = 0;
  d.pad = 0;
  return d;
}

// 1-D bulk copy global -> shared, completion counted on an mbarrier (addresses and size multiples of 16).
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__global__ void __launch_bounds__(kDecThreads, 2)
decode_attn_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_k16,
                   const __grid_constant__ CUtensorMap map_v16) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int G = p.G, Hkv = p.Hkv;
  unsigned char* stages = smem;
  __nv_bfloat16* s_q = reinterpret_cast<__nv_bfloat16*>(smem + kDecStages * kStageBytes);          // [kSegRing][G][128]
  float* merge_o = reinterpret_cast<float*>(s_q + kSegRing * G * 128);                            // [n_merge][4][G][128]
  float* merge_ml = merge_o + p.n_merge * kDecConsumerWarps * G * 128;                              // [n_merge][4][G][2]
  int* s_prefix = reinterpret_cast<int*>(merge_ml + p.n_merge * kDecConsumerWarps * G * 2);       // [batch + 1]
  __shared__ __align__(8) uint64_t bar_full[kDecStages];
  __shared__ __align__(8) uint64_t bar_empty[kDecStages];
  __shared__ __align__(8) uint64_t bar_merge_full[2];
  __shared__ __align__(8) uint64_t bar_merge_empty[2];
  __shared__ __align__(16) SegDesc s_desc[kSegRing];
  __shared__ __align__(16) SegDesc s_merge_desc[2];
  __shared__ __align__(16) SegDesc s_pending[kDecPending];
  __shared__ int s_warp_sums[kDecThreads / 32];
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int max_len = p.bt_cols * p.block_size;

  if (tid == 0) {
    s_abort = 0;
    for (int s = 0; s < kDecStages; ++s) {
      mbar_init(&bar_full[s], 1);
      mbar_init(&bar_empty[s], kDecConsumerWarps);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bar_merge_full[s], kDecConsumerWarps);
      mbar_init(&bar_merge_empty[s], 1);
    }
    mbar_fence_init();
  }

  // Launched with programmatic stream serialization: the kernel may start while the previous kernel
  // of the stream is still running, if that kernel allows it (griddepcontrol.launch_dependents; only
  // this library's store and producer kernels do, any other kernel has completed before this one
  // starts).  Those kernels write K/V rows of the cache and the query rows, never the metadata, so
  // the scan over context_lens, the piece geometry and the first block-table reads below run ahead;
  // every thread that goes on to touch q, the cache, the output or the workspace first executes
  // griddepcontrol.wait (the consumer warps only ever read shared memory filled after it).

  // ---- tile counts per sequence and their exclusive prefix (block scan) ----
  {
    const int per = (p.batch + kDecThreads - 1) / kDecThreads;
    const int i0 = tid * per;
    int local[kDecPer];
    int sum = 0;
#pragma unroll
    for (int k = 0; k < kDecPer; ++k) {
      int nt = 0;
      const int i = i0 + k;
      if (k < per && i < p.batch) {
        int len = p.context_lens[i];
        len = len < 0 ? 0 : (len > max_len ? max_len : len);
        nt = (len + kTile - 1) / kTile;
      }
      local[k] = nt;
      sum += nt;
    }
    int incl = sum;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += v;
    }
    if (lane == 31) s_warp_sums[warp] = incl;
    __syncthreads();
    int excl = incl - sum;
    for (int w = 0; w < warp; ++w) excl += s_warp_sums[w];
#pragma unroll
    for (int k = 0; k < kDecPer; ++k) {
      const int i = i0 + k;
      if (k < per && i < p.batch) {
        s_prefix[i] = excl;
        excl += local[k];
        if (i == p.batch - 1) s_prefix[p.batch] = excl;
      }
    }
    __syncthreads();
  }

  // ---- sequences with no context produce zeros (the epilogue warp's job, before anything else) ----
  if (warp == kDecEpilogueWarp) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    for (int i = blockIdx.x; i < p.batch; i += gridDim.x) {
      if (s_prefix[i + 1] == s_prefix[i]) {
        uint4* o = reinterpret_cast<uint4*>(p.out + static_cast<long long>(i) * p.H * 128);
        for (int v = lane; v < p.H * 16; v += 32) o[v] = make_uint4(0, 0, 0, 0);
      }
    }
  }

  const long long T = static_cast<long long>(s_prefix[p.batch]) * Hkv;  // tiles in this launch
  const DecPieces pc = dec_pieces(T, static_cast<int>(gridDim.x), p.dyn_factor, p.big_pct, p.small_pct100, p.small_n);
  const int cta = blockIdx.x;
  if (cta >= pc.g) return;

  volatile int* abort_flag = &s_abort;

  if (warp == kDecProducerWarp) {
    // =========================== producer warp ===========================
    if (lane != 0) return;
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    tma_prefetch_desc(&map_k16);
    tma_prefetch_desc(&map_v16);
    int it = 0, segc = 0;
    bool ok = true;
    int piece = cta;   // the CTA's own static piece first, then tickets
    long long r_begin = pc.start(piece), r_end = pc.start(piece + 1);
    SegDesc cur = dec_locate(s_prefix, p.batch, Hkv, r_begin, r_begin, r_end, piece);
    // metadata of a segment, fetched one segment ahead: its length and its first two block ids
    int cur_len = p.context_lens[cur.seq];
    const int* cur_bt = p.block_tables + cur.seq * p.bt_row_stride;
    int cur_col0 = (cur.t0 * kTile) / p.block_size;
    int cur_blk0 = cur_bt[cur_col0];
    int cur_blk1 = cur_col0 + 1 < p.bt_cols ? cur_bt[cur_col0 + 1] : -1;
    asm volatile("griddepcontrol.wait;" ::: "memory");   // from here on: query rows and the cache
    while (true) {
      cur_len = cur_len > max_len ? max_len : cur_len;
      cur.len = cur_len;
      const int last_col = (cur_len - 1) / p.block_size;
      int col_now = cur_col0;
      long long blk_now = cur_blk0;
      long long blk_next = cur_col0 < last_col ? cur_blk1 : -1;
      SegDesc nxt;
      nxt.seq = -1;
      int nxt_len = 0, nxt_col0 = 0, nxt_blk0 = -1, nxt_blk1 = -1;
      const int* nxt_bt = nullptr;
      for (int t = cur.t0; t < cur.t1; ++t, ++it) {
        const int stage = it % kDecStages;
        const uint32_t ph = (it / kDecStages) & 1;
        if (!mbar_wait(&bar_empty[stage], ph ^ 1, abort_flag)) { ok = false; break; }
        const int tok0 = t * kTile;
        const int col = tok0 / p.block_size;
        if (col != col_now) {
          col_now = col;
          blk_now = blk_next;
          blk_next = col_now < last_col ? cur_bt[col_now + 1] : -1;
        }
        int slot0 = -kTile;  // out-of-range block id: the box lies outside the tensor and reads zeros
        if (blk_now >= 0 && blk_now < p.num_blocks)
          slot0 = static_cast<int>(blk_now * p.block_size + (tok0 - col * p.block_size));
        unsigned char* st = stages + stage * kStageBytes;
        const int valid = cur_len - tok0;
        const int nslab = valid >= kTile - 15 ? 4 : (valid + 15) >> 4;
        uint32_t tx = nslab == 4 ? kStageBytes : nslab * 4 * 2048;
        const bool first = t == cur.t0;
        if (first) {
          // descriptor and query rows travel with the segment's first tile
          s_desc[segc % kSegRing] = cur;
          tx += G * 256;
        }
        mbar_expect_tx(&bar_full[stage], tx);
        if (first)
          bulk_load_1d(s_q + (segc % kSegRing) * G * 128,
                       p.q + cur.seq * p.q_row_stride + static_cast<long long>(cur.h) * G * 128, G * 256, &bar_full[stage]);
        if (nslab == 4) {
          tma_load_3d(st, &map_k, &bar_full[stage], 0, cur.h, slot0);
          tma_load_3d(st + kSubTileBytes, &map_k, &bar_full[stage], 64, cur.h, slot0);
          tma_load_3d(st + 2 * kSubTileBytes, &map_v, &bar_full[stage], 0, cur.h, slot0);
          tma_load_3d(st + 3 * kSubTileBytes, &map_v, &bar_full[stage], 64, cur.h, slot0);
        } else {
          // ragged last tile of the sequence: fetch only the 16-token slabs that hold tokens
          for (int sl = 0; sl < nslab; ++sl) {
            unsigned char* d = st + sl * 2048;
            tma_load_3d(d, &map_k16, &bar_full[stage], 0, cur.h, slot0 + sl * 16);
            tma_load_3d(d + kSubTileBytes, &map_k16, &bar_full[stage], 64, cur.h, slot0 + sl * 16);
            tma_load_3d(d + 2 * kSubTileBytes, &map_v16, &bar_full[stage], 0, cur.h, slot0 + sl * 16);
            tma_load_3d(d + 3 * kSubTileBytes, &map_v16, &bar_full[stage], 64, cur.h, slot0 + sl * 16);
          }
        }
        if (first) {
          // with this segment under way, find the next one and start fetching its metadata
          long long x = cur.seg_start + cur.t1;   // flat position after this segment's part
          if (x >= r_end) {
            // next piece: a ticket.  Each of the g CTAs draws until it fails, so exactly
            // dynamic() + g tickets are drawn per launch; whoever draws the last one resets the counter.
            int np = -1;
            if (pc.dynamic() > 0) {
              const unsigned int tk = atomicAdd(p.ticket, 1u);
              if (tk == static_cast<unsigned int>(pc.dynamic() + pc.g - 1)) atomicExch(p.ticket, 0u);
              if (tk < static_cast<unsigned int>(pc.dynamic())) np = pc.g + static_cast<int>(tk);
            }
            if (np >= 0) {
              piece = np;
              r_begin = pc.start(np);
              r_end = pc.start(np + 1);
              x = r_begin;
            } else {
              x = -1;
            }
          }
          if (x >= 0) {
            nxt = dec_locate(s_prefix, p.batch, Hkv, x, r_begin, r_end, piece);
            nxt_len = p.context_lens[nxt.seq];
            nxt_bt = p.block_tables + nxt.seq * p.bt_row_stride;
            nxt_col0 = (nxt.t0 * kTile) / p.block_size;
            nxt_blk0 = nxt_bt[nxt_col0];
            nxt_blk1 = nxt_col0 + 1 < p.bt_cols ? nxt_bt[nxt_col0 + 1] : -1;
          }
        }
      }
      if (!ok) break;
      ++segc;
      if (nxt.seq < 0) break;
      cur = nxt;
      cur_len = nxt_len;
      cur_bt = nxt_bt;
      cur_col0 = nxt_col0;
      cur_blk0 = nxt_blk0;
      cur_blk1 = nxt_blk1;
    }
    if (ok) {
      // end marker: a descriptor with seq = -1 on the next full-barrier, no bytes attached
      const int stage = it % kDecStages;
      const uint32_t ph = (it / kDecStages) & 1;
      if (mbar_wait(&bar_empty[stage], ph ^ 1, abort_flag)) {
        s_desc[segc % kSegRing].seq = -1;
        mbar_arrive(&bar_full[stage]);
      }
    } else {
      atomicExch(&g_status_decode, 1);
    }
    return;
  }

  if (warp == kDecEpilogueWarp) {
    // =========================== epilogue warp ===========================
    // Lane owns 4 of the 128 output dims.  Step 1 for every segment: combine the four consumer
    // warps' states and store the row (or the partial) -- no waiting on global memory, so the
    // consumers get their hand-off buffer back at once.  The slow part of a partial (fence, arrival
    // counter, merge: several dependent trips to L2) is queued and flushed when no hand-off is
    // waiting; one fence and one round of atomics then serve every queued partial.
    int n_pending = 0;
    auto flush = [&]() {
      if (n_pending == 0) return;
      __threadfence();
      __syncwarp();
      int expected = 0, old = -1;
      if (lane < n_pending) {
        const SegDesc& d = s_pending[lane];
        expected = pc.of(d.seg_start + d.nt - 1) - pc.of(d.seg_start);
        old = atomicAdd(&p.counters[d.seq * Hkv + d.h], 1);
      }
      const unsigned last_mask = __ballot_sync(0xffffffffu, lane < n_pending && old == expected);
      if (last_mask) __threadfence();
      for (int k = 0; k < n_pending; ++k) {
        if (!((last_mask >> k) & 1u)) continue;
        // this CTA brought the last partial of (sequence, head) k: merge them all
        const SegDesc d = s_pending[k];
        const int i_first = pc.of(d.seg_start);
        const int n = pc.of(d.seg_start + d.nt - 1) - i_first + 1;
        if (n <= 4) {
          // The common case (a few partials): all loads of a query head are issued before the first is used,
          // one trip to L2 per head instead of two.
          int sl[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int i = i_first + (u < n ? u : 0);
            sl[u] = i * 2 + (d.seg_start <= pc.start(i) ? 0 : 1);
          }
#pragma unroll 1
          for (int gq = 0; gq < G; ++gq) {
            float4 v[4];
            float2 ml[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (u < n) {
                v[u] = __ldcg(reinterpret_cast<const float4*>(p.ws_o + (static_cast<long long>(sl[u]) * G + gq) * 128 + lane * 4));
                ml[u] = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + (sl[u] * G + gq) * 2));
              }
            }
            float M = -INFINITY;
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (u < n) M = fmaxf(M, ml[u].x);
            float L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              if (u < n) {
                const float wu = fast_exp2(ml[u].x - M);
                L += ml[u].y * wu;
                acc.x += v[u].x * wu; acc.y += v[u].y * wu; acc.z += v[u].z * wu; acc.w += v[u].w * wu;
              }
            }
            const float inv = 1.f / L;
            uint2 o2;
            o2.x = pack_bf16(acc.x * inv, acc.y * inv);
            o2.y = pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(p.out + (static_cast<long long>(d.seq) * p.H + d.h * G + gq) * 128 + lane * 4) = o2;
          }
        } else {
          for (int gq = 0; gq < G; ++gq) {
            float M = -INFINITY, L = 0.f;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int base = 0; base < n; base += 32) {
              const int cnt = n - base < 32 ? n - base : 32;
              // lane j looks after partial base + j: its slot, its (max, sum)
              int sl = 0;
              float mj = -INFINITY, lj = 0.f;
              if (lane < cnt) {
                const int i = i_first + base + lane;
                sl = i * 2 + (d.seg_start <= pc.start(i) ? 0 : 1);
                const float2 v = __ldcg(reinterpret_cast<const float2*>(p.ws_ml + (sl * G + gq) * 2));
                mj = v.x;
                lj = v.y;
              }
              float Mr = mj;
  #pragma unroll
              for (int off = 16; off > 0; off >>= 1) Mr = fmaxf(Mr, __shfl_xor_sync(0xffffffffu, Mr, off));
              const float Mn = fmaxf(M, Mr);
              const float rescale = fast_exp2(M - Mn);
              const float wj = fast_exp2(mj - Mn);
              float Lr = lj * wj;
  #pragma unroll
              for (int off = 16; off > 0; off >>= 1) Lr += __shfl_xor_sync(0xffffffffu, Lr, off);
              L = L * rescale + Lr;
              acc.x *= rescale; acc.y *= rescale; acc.z *= rescale; acc.w *= rescale;
              M = Mn;
              // every lane accumulates its 4 dims over the partials, 8 independent loads at a time
              for (int u0 = 0; u0 < cnt; u0 += 8) {
                float4 v[8];
  #pragma unroll
                for (int u = 0; u < 8; ++u) {
                  const int slu = __shfl_sync(0xffffffffu, sl, (u0 + u) & 31);
                  if (u0 + u < cnt)
                    v[u] = __ldcg(reinterpret_cast<const float4*>(p.ws_o + (static_cast<long long>(slu) * G + gq) * 128 + lane * 4));
                }
  #pragma unroll
                for (int u = 0; u < 8; ++u) {
                  const float wu = __shfl_sync(0xffffffffu, wj, (u0 + u) & 31);
                  if (u0 + u < cnt) { acc.x += v[u].x * wu; acc.y += v[u].y * wu; acc.z += v[u].z * wu; acc.w += v[u].w * wu; }
                }
              }
            }
            const float inv = 1.f / L;
            uint2 o2;
            o2.x = pack_bf16(acc.x * inv, acc.y * inv);
            o2.y = pack_bf16(acc.z * inv, acc.w * inv);
            *reinterpret_cast<uint2*>(p.out + (static_cast<long long>(d.seq) * p.H + d.h * G + gq) * 128 + lane * 4) = o2;
          }
        }
        if (lane == 0) p.counters[d.seq * Hkv + d.h] = 0;
      }
      __syncwarp();
      n_pending = 0;
    };
    // (flush() is expanded in one place only: it is large, and three copies cost the kernel registers)
    bool finished = false, flush_now = false;
    for (int n = 0;;) {
      const int e = n % p.n_merge;
      const uint32_t ph = (n / p.n_merge) & 1;
      const bool ready = !finished && !flush_now && mbar_try_wait(&bar_merge_full[e], ph);
      flush_now = false;
      if (!ready) {
        flush();                                     // nothing to combine right now: do the slow part
        if (finished) break;
        if (!mbar_wait(&bar_merge_full[e], ph, abort_flag)) break;
      }
      const SegDesc d = s_merge_desc[e];
      if (d.seq < 0) { finished = true; continue; }
      const float* mo = merge_o + e * kDecConsumerWarps * G * 128;
      const float* ml = merge_ml + e * kDecConsumerWarps * G * 2;
      const bool full = d.t0 == 0 && d.t1 == d.nt;
      for (int gq = 0; gq < G; ++gq) {
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kDecConsumerWarps; ++w) M = fmaxf(M, ml[(w * G + gq) * 2]);
        float L = 0.f;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < kDecConsumerWarps; ++w) {
          const float wgt = fast_exp2(ml[(w * G + gq) * 2] - M);
          L += ml[(w * G + gq) * 2 + 1] * wgt;
          const float4 v = *reinterpret_cast<const float4*>(mo + (w * G + gq) * 128 + lane * 4);
          acc.x += v.x * wgt; acc.y += v.y * wgt; acc.z += v.z * wgt; acc.w += v.w * wgt;
        }
        if (full) {
          const float inv = 1.f / L;
          uint2 o2;
          o2.x = pack_bf16(acc.x * inv, acc.y * inv);
          o2.y = pack_bf16(acc.z * inv, acc.w * inv);
          *reinterpret_cast<uint2*>(p.out + (static_cast<long long>(d.seq) * p.H + d.h * G + gq) * 128 + lane * 4) = o2;
        } else {
          *reinterpret_cast<float4*>(p.ws_o + (static_cast<long long>(d.slot) * G + gq) * 128 + lane * 4) = acc;
          if (lane == 0) *reinterpret_cast<float2*>(p.ws_ml + (d.slot * G + gq) * 2) = make_float2(M, L);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_merge_empty[e]);   // the consumers may refill the hand-off buffer
      ++n;
      if (!full) {
        if (lane == 0) s_pending[n_pending] = d;
        __syncwarp();
        if (++n_pending == kDecPending) flush_now = true;   // a full queue is flushed at the top of the loop
      }
    }
    return;
  }

  // ============================= consumer warps =============================
  const int row = lane >> 2;        // A/C fragment row (query head within the kv group)
  const int quad = lane & 3;
  const bool row0_ok = row < G, row1_ok = row + 8 < G;
  int it = 0, segc = 0;
  bool ok = true;
  while (ok) {
    // ---- a new segment: its descriptor and query rows arrive with its first tile ----
    {
      const int stage = it % kDecStages;
      const uint32_t ph = (it / kDecStages) & 1;
      if (!mbar_wait(&bar_full[stage], ph, abort_flag)) { ok = false; break; }
    }
    const SegDesc d = s_desc[segc % kSegRing];
    if (d.seq < 0) break;
    uint32_t qa[8][4];   // query fragments: rows = the G heads sharing the kv head
    {
      const uint32_t* q0 = reinterpret_cast<const uint32_t*>(s_q + (segc % kSegRing) * G * 128 + row * 128);
      const uint32_t* q1 = q0 + 8 * 64;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qa[ks][0] = row0_ok ? q0[ks * 8 + quad] : 0u;
        qa[ks][1] = row1_ok ? q1[ks * 8 + quad] : 0u;
        qa[ks][2] = row0_ok ? q0[ks * 8 + 4 + quad] : 0u;
        qa[ks][3] = row1_ok ? q1[ks * 8 + 4 + quad] : 0u;
      }
    }
    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int t = d.t0; t < d.t1; ++t, ++it) {
      const int stage = it % kDecStages;
      const uint32_t ph = (it / kDecStages) & 1;
      if (t != d.t0 && !mbar_wait(&bar_full[stage], ph, abort_flag)) { ok = false; break; }
      const int valid = d.len - (t * kTile + warp * 16);  // valid tokens in this warp's 16-token slab
      if (valid > 0) {
        const uint32_t st = smem_u32(stages + stage * kStageBytes);
        const uint32_t k_base = st, v_base = st + 2 * kSubTileBytes;
        if (valid < 16) {
          // rows past the sequence end hold whatever the cache block holds: zero the V rows so
          // that 0 * garbage cannot produce NaN (K garbage is masked by select below)
          unsigned char* vb = stages + stage * kStageBytes + 2 * kSubTileBytes;
          for (int e = lane; e < 16 * 16; e += 32) {
            const int r = warp * 16 + (e >> 4), c = e & 15;
            if ((e >> 4) >= valid)
              *reinterpret_cast<uint4*>(vb + (c >> 3) * kSubTileBytes + r * 128 + (((c & 7) ^ (r & 7)) << 4)) =
                  make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
        }
        // ---- S = Q K^T (16 x 16 tokens) ----
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
        {
          const int tok = warp * 16 + ((lane >> 4) << 3) + (lane & 7);
          const int dsel = ((lane >> 3) & 1) << 3;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(k_base + tile_offset(tok, ks * 16 + dsel, kTile), b0, b1, b2, b3);
            mma_bf16_16816(s[0], qa[ks], b0, b1);
            mma_bf16_16816(s[1], qa[ks], b2, b3);
          }
        }
        // ---- online softmax (log2 domain) ----
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const bool in = (j * 8 + quad * 2 + e) < valid;
            s[j][e] = in ? s[j][e] * p.scale_log2 : -INFINITY;
            s[j][2 + e] = in ? s[j][2 + e] * p.scale_log2 : -INFINITY;
            mx0 = fmaxf(mx0, s[j][e]);
            mx1 = fmaxf(mx1, s[j][2 + e]);
          }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float a0 = fast_exp2(m0 - mn0), a1 = fast_exp2(m1 - mn1);
        m0 = mn0; m1 = mn1;
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            s[j][e] = fast_exp2(s[j][e] - mn0);
            s[j][2 + e] = fast_exp2(s[j][2 + e] - mn1);
            ps0 += s[j][e];
            ps1 += s[j][2 + e];
          }
        }
        l0 = l0 * a0 + ps0;
        l1 = l1 * a1 + ps1;
        if (a0 != 1.f || a1 != 1.f) {
#pragma unroll
          for (int n = 0; n < 16; ++n) { o[n][0] *= a0; o[n][1] *= a0; o[n][2] *= a1; o[n][3] *= a1; }
        }
        // ---- O += P V ----
        uint32_t pa[4];
        pa[0] = pack_bf16(s[0][0], s[0][1]);
        pa[1] = pack_bf16(s[0][2], s[0][3]);
        pa[2] = pack_bf16(s[1][0], s[1][1]);
        pa[3] = pack_bf16(s[1][2], s[1][3]);
        {
          const int tok = warp * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
          const int dsel = (lane >> 4) << 3;
#pragma unroll
          for (int n2 = 0; n2 < 8; ++n2) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4_trans(v_base + tile_offset(tok, n2 * 16 + dsel, kTile), b0, b1, b2, b3);
            mma_bf16_16816(o[2 * n2], pa, b0, b1);
            mma_bf16_16816(o[2 * n2 + 1], pa, b2, b3);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_empty[stage]);
    }
    if (!ok) break;

    // ---- hand the warp's running state to the epilogue warp and move on ----
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    {
      const int e = segc % p.n_merge;
      const uint32_t ph = (segc / p.n_merge) & 1;
      if (!mbar_wait(&bar_merge_empty[e], ph ^ 1, abort_flag)) { ok = false; break; }
      float* mo = merge_o + (e * kDecConsumerWarps + warp) * G * 128;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        if (row0_ok) *reinterpret_cast<float2*>(mo + row * 128 + n * 8 + quad * 2) = make_float2(o[n][0], o[n][1]);
        if (row1_ok) *reinterpret_cast<float2*>(mo + (row + 8) * 128 + n * 8 + quad * 2) = make_float2(o[n][2], o[n][3]);
      }
      if (quad == 0) {
        float* ml = merge_ml + (e * kDecConsumerWarps + warp) * G * 2;
        if (row0_ok) { ml[row * 2] = m0; ml[row * 2 + 1] = l0; }
        if (row1_ok) { ml[(row + 8) * 2] = m1; ml[(row + 8) * 2 + 1] = l1; }
      }
      if (tid == 0) s_merge_desc[e] = d;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_merge_full[e]);
    }
    ++segc;
  }
  // tell the epilogue warp that nothing more will come
  if (ok) {
    const int e = segc % p.n_merge;
    const uint32_t ph = (segc / p.n_merge) & 1;
    if (mbar_wait(&bar_merge_empty[e], ph ^ 1, abort_flag)) {
      if (tid == 0) s_merge_desc[e].seq = -1;
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_merge_full[e]);
    }
  } else if (lane == 0) {
    atomicExch(&g_status_decode, 1);
  }
}


int read_status_decode() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_status_decode, sizeof(int));
  return v;
}

// Only the status word lives in the library; the ticket and arrival counters of an abandoned launch
// are in the caller's workspace, which the caller has to zero-fill again.
int reset_state_decode() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_status_decode, &zero, sizeof(int)), "device_status: clearing the decode status word");
}

// Two hand-off buffers between consumers and the epilogue warp when two CTAs still fit on an SM with them.
static int decode_merge_buffers(int G) { return G <= 2 ? 2 : 1; }

static size_t decode_smem_bytes(int G) {
  return 1024 + static_cast<size_t>(kDecStages) * kStageBytes + static_cast<size_t>(kSegRing) * G * 256 +
         static_cast<size_t>(decode_merge_buffers(G)) * kDecConsumerWarps * G * 130 * 4 + (kDecMaxBatch + 1) * 4 + 64;
}

static int decode_grid() { return 2 * sm_count(); }

// Two partial slots per piece; at most grid static + grid big + 4 * grid small pieces.
static long long decode_partial_slots(int grid) { return 12LL * grid; }
static long long decode_partial_bytes(int grid, int G) { return decode_partial_slots(grid) * G * 130 * 4; }
static long long decode_ws_bytes(int grid, int G) {
  return kWsStatusBytes + static_cast<long long>(kWsCounterInts) * 4 + decode_partial_bytes(grid, G);
}

}  // namespace b200

extern "C" int64_t b200_decode_workspace_bytes(int32_t max_batch, int32_t num_heads, int32_t num_kv_heads,
                                               int32_t head_dim) {
  using namespace b200;
  if (max_batch <= 0 || num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads || head_dim != 128)
    return set_error(kErrBadShape, "decode_workspace_bytes: bad geometry (batch=%d H=%d Hkv=%d D=%d)", max_batch,
                     num_heads, num_kv_heads, head_dim);
  const int grid = decode_grid();
  if (grid <= 0) return set_error(kErrNoDriver, "decode_workspace_bytes: no CUDA device");
  if (num_kv_heads > 128 || num_heads / num_kv_heads > kMaxG)
    return set_error(kErrBadShape, "decode_workspace_bytes: at most 128 kv heads and %d query heads per kv head", kMaxG);
  return decode_ws_bytes(grid, num_heads / num_kv_heads);
}

extern "C" int b200_decode_attn(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                int64_t num_blocks, int32_t block_size, const int32_t* block_tables,
                                int64_t bt_row_stride, int32_t bt_cols, const int32_t* context_lens, void* out,
                                void* workspace, int64_t workspace_bytes, int32_t batch, int32_t num_heads,
                                int32_t num_kv_heads, int32_t head_dim, float scale, void* stream) {
  using namespace b200;
  if (batch < 0) return set_error(kErrBadShape, "decode_attn: negative batch");
  if (batch == 0) return kOk;
  if (!q || !k_cache || !v_cache || !block_tables || !context_lens || !out)
    return set_error(kErrNullPointer, "decode_attn: null pointer argument");
  if (head_dim != 128) return set_error(kErrBadShape, "decode_attn: head_dim must be 128 (got %d)", head_dim);
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads)
    return set_error(kErrBadShape, "decode_attn: num_heads (%d) must be a positive multiple of num_kv_heads (%d)",
                     num_heads, num_kv_heads);
  const int G = num_heads / num_kv_heads;
  if (G > kMaxG) return set_error(kErrBadShape, "decode_attn: at most %d query heads per kv head (got %d)", kMaxG, G);
  if (num_kv_heads > 128) return set_error(kErrBadShape, "decode_attn: at most 128 kv heads (got %d)", num_kv_heads);
  if (block_size <= 0 || block_size % 256)
    return set_error(kErrBadShape, "decode_attn: block_size must be a positive multiple of 256 (got %d)", block_size);
  if (num_blocks <= 0 || num_blocks * block_size >= (1LL << 31))
    return set_error(kErrBadShape, "decode_attn: num_blocks * block_size must be in (0, 2^31)");
  if (bt_cols <= 0 || bt_row_stride < bt_cols || static_cast<long long>(bt_cols) * block_size >= (1LL << 30))
    return set_error(kErrBadShape, "decode_attn: bad block table geometry (cols=%d stride=%lld)", bt_cols,
                     (long long)bt_row_stride);
  if (q_row_stride < static_cast<long long>(num_heads) * 128 || q_row_stride % 8)
    return set_error(kErrMisaligned, "decode_attn: q_row_stride must be >= H*128 and a multiple of 8 elements");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return set_error(kErrMisaligned, "decode_attn: q, caches and out must be 16-byte aligned");
  const int grid = decode_grid();
  if (grid <= 0) return set_error(kErrNoDriver, "decode_attn: no CUDA device");
  const long long need = decode_ws_bytes(grid, G);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return set_error(kErrWorkspace, "decode_attn: workspace of %lld bytes (16-byte aligned, zero-filled once) required, got %lld",
                     need, (long long)workspace_bytes);

  CUtensorMap map_k, map_v;
  int rc = make_tokens_heads_map(&map_k, k_cache, static_cast<uint64_t>(num_blocks) * block_size, num_kv_heads,
                                 static_cast<uint64_t>(num_kv_heads) * 128, kTile);
  if (rc) return rc;
  rc = make_tokens_heads_map(&map_v, v_cache, static_cast<uint64_t>(num_blocks) * block_size, num_kv_heads,
                             static_cast<uint64_t>(num_kv_heads) * 128, kTile);
  if (rc) return rc;
  CUtensorMap map_k16, map_v16;   // 16-token boxes for the ragged last tile of a sequence
  rc = make_tokens_heads_map(&map_k16, k_cache, static_cast<uint64_t>(num_blocks) * block_size, num_kv_heads,
                             static_cast<uint64_t>(num_kv_heads) * 128, 16);
  if (rc) return rc;
  rc = make_tokens_heads_map(&map_v16, v_cache, static_cast<uint64_t>(num_blocks) * block_size, num_kv_heads,
                             static_cast<uint64_t>(num_kv_heads) * 128, 16);
  if (rc) return rc;

  const size_t smem = decode_smem_bytes(G);
  static std::atomic<size_t> configured[kMaxDevices];
  rc = ensure_dynamic_smem(reinterpret_cast<const void*>(decode_attn_kernel), smem, configured, "decode_attn: cudaFuncSetAttribute");
  if (rc) return rc;

  unsigned char* ws = static_cast<unsigned char*>(workspace);
  DecodeParams p;
  p.bt_row_stride = bt_row_stride;
  p.bt_cols = bt_cols;
  p.H = num_heads;
  p.Hkv = num_kv_heads;
  p.G = G;
  p.block_size = block_size;
  p.num_blocks = num_blocks;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.n_merge = decode_merge_buffers(G);
  p.dyn_factor = kDynFactor;
  p.big_pct = kDynBigPct;
  p.small_pct100 = kDynSmallPct100;
  p.small_n = kDynSmallN;
  p.ticket = reinterpret_cast<unsigned int*>(ws);
  p.counters = reinterpret_cast<int*>(ws + kWsStatusBytes);
  p.ws_o = reinterpret_cast<float*>(ws + kWsStatusBytes + static_cast<long long>(kWsCounterInts) * 4);
  p.ws_ml = p.ws_o + decode_partial_slots(grid) * G * 128;
  p.q_row_stride = q_row_stride;
  for (int b0 = 0; b0 < batch; b0 += kDecMaxBatch) {
    p.batch = batch - b0 < kDecMaxBatch ? batch - b0 : kDecMaxBatch;
    p.q = static_cast<const __nv_bfloat16*>(q) + b0 * q_row_stride;
    p.out = static_cast<__nv_bfloat16*>(out) + static_cast<long long>(b0) * num_heads * 128;
    p.context_lens = context_lens + b0;
    p.block_tables = block_tables + b0 * bt_row_stride;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t le = cudaLaunchKernelEx(&cfg, decode_attn_kernel, p, map_k, map_v, map_k16, map_v16);
    g_launches.fetch_add(1);
    rc = check_cuda(le != cudaSuccess ? le : cudaGetLastError(), "decode_attn launch");
    if (rc) return rc;
  }
  return kOk;
}

// ---------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// Some hosts of this library have nowhere to get a workspace from: a serving engine that has
// already handed every free byte of the GPU to its KV cache (nano-vllm sizes the cache from the
// free memory it finds, so a later cudaMalloc can fail), a plugin slot whose contract forbids
// allocation inside the call, or code that runs where the framework's caching allocator must not
// be touched.  For them the scratch of the decode kernel lives in the library image itself: a
// file-scope __device__ array that every GPU loading the library holds until the process exits.
// ---------------------------------------------------------------------------------------------
namespace b200 {

constexpr int kStaticMaxGridTimesG = 320 * 4;   // persistent CTAs x query heads per kv head the scratch has room for
constexpr long long kStaticScratchBytes =
    kWsStatusBytes + static_cast<long long>(kWsCounterInts) * 4 + 12LL * kStaticMaxGridTimesG * 130 * 4;

static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

// Device address of the array above on the current device.  In host code the array's name is only a
// handle for the runtime, never an address a kernel may be given, so the address is asked for
// once per device (with that device current) and remembered.
static int static_scratch_address(void** out) {
  static void* cached[64];
  static std::atomic<int> ready[64];
  int dev = 0;
  int rc = check_cuda(cudaGetDevice(&dev), "decode_attn_static: cudaGetDevice");
  if (rc) return rc;
  if (dev < 0 || dev >= 64) return set_error(kErrDevice, "decode_attn_static: device ordinal %d not supported", dev);
  if (!ready[dev].load(std::memory_order_acquire)) {
    void* ptr = nullptr;
    rc = check_cuda(cudaGetSymbolAddress(&ptr, g_decode_static_scratch), "decode_attn_static: cudaGetSymbolAddress");
    if (rc) return rc;
    if (!ptr) return set_error(kErrDevice, "decode_attn_static: the scratch array has no address on device %d", dev);
    cached[dev] = ptr;
    ready[dev].store(1, std::memory_order_release);
  }
  *out = cached[dev];
  return kOk;
}

}  // namespace b200

extern "C" int64_t b200_decode_static_scratch_bytes(void) { return b200::kStaticScratchBytes; }

extern "C" int b200_decode_attn_static(const void* q, int64_t q_row_stride, const void* k_cache, const void* v_cache,
                                       int64_t num_blocks, int32_t block_size, const int32_t* block_tables,
                                       int64_t bt_row_stride, int32_t bt_cols, const int32_t* context_lens, void* out,
                                       int32_t batch, int32_t num_heads, int32_t num_kv_heads, int32_t head_dim,
                                       float scale, void* stream) {
  using namespace b200;
  if (batch < 0) return set_error(kErrBadShape, "decode_attn_static: negative batch");
  if (batch == 0) return kOk;
  if (num_heads <= 0 || num_kv_heads <= 0 || num_heads % num_kv_heads)
    return set_error(kErrBadShape, "decode_attn_static: num_heads (%d) must be a positive multiple of num_kv_heads (%d)",
                     num_heads, num_kv_heads);
  const int grid = decode_grid();
  if (grid <= 0) return set_error(kErrNoDriver, "decode_attn_static: no CUDA device");
  const int G = num_heads / num_kv_heads;
  if (static_cast<long long>(grid) * G > kStaticMaxGridTimesG || num_kv_heads > 128)
    return set_error(kErrWorkspace,
                     "decode_attn_static: %d persistent CTAs x %d query heads per kv head exceeds the built-in scratch's "
                     "limit of %d (and kv heads must be <= 128); use b200_decode_attn with a caller-owned workspace",
                     grid, G, kStaticMaxGridTimesG);
  void* scratch = nullptr;
  int rc = static_scratch_address(&scratch);
  if (rc) return rc;
  // The array keeps whatever the previous call left.  Partials are always written before they are
  // read; the ticket counter and the arrival counters are what must start at zero, so clear them here.
  const long long per_launch = batch < kDecMaxBatch ? batch : kDecMaxBatch;
  rc = check_cuda(cudaMemsetAsync(scratch, 0, kWsStatusBytes + static_cast<size_t>(per_launch) * num_kv_heads * 4,
                                  static_cast<cudaStream_t>(stream)),
                  "decode_attn_static: clearing the counters");
  if (rc) return rc;
  return b200_decode_attn(q, q_row_stride, k_cache, v_cache, num_blocks, block_size, block_tables, bt_row_stride, bt_cols,
                          context_lens, out, scratch, kStaticScratchBytes, batch, num_heads, num_kv_heads, head_dim,
                          scale, stream);
}
