// Single-token GQA decode, sm_100a: a TMA producer warp that streams K/V tiles ahead of the math
// warps, across work-item boundaries.
//
// Role in the reference: the same as gqa_decode.cu (GQADecodeKernel / GQADecodePagedKernel and their
// split-KV combine, src/tileops/kernels/attention/gqa_decode.py:23-306, gqa_decode_paged.py:44-395 in
// tile-ai/TileOPs); the producer / consumer split is what the reference's Hopper batch-1 kernels do
// with a TMA warp and a consumer warpgroup (gqa_decode_bs1_common.py:57-292), here for any batch.
//
// Why a second kernel: in gqa_decode.cu the math warps issue their own cp.async gathers, so the
// load pipeline drains at the end of every work item and refills at the start of the next; on
// ragged batches that is the largest loss.  Here
//   * warp 4 owns the shared-memory ring: per 64-token tile it issues one TMA box per 128-byte panel
//     of K and of V (swizzled, no padding), waits only for a free stage, and walks the CTA's items
//     back to back, so the next item's first tiles are in flight while the math warps finish the
//     current one; it also copies each item's q rows into shared memory and reads the block-table
//     entries (32 tiles per global read, one lane each);
//   * warps 0-3 are the math warps of gqa_decode.cu (tokens on the MMA M dimension, q heads on N = 8,
//     mma.sync.m16n8k16, movmatrix for P^T, FP8 expanded with cvt.rn.f16x2.e4m3x2), without a single
//     load instruction or address computation for K/V; stages go back to the producer through mbarriers
//     (one arrival per warp, after the MMAs that consumed the stage); the four warps meet once per item in
//     an 8.7 KB area of its own, half of the head dims at a time, at an mbarrier at which every thread
//     arrives (an arrival releases only the arriving thread's stores).
// Served layouts: 64-token tiles that are one copy (no block table, or page_size % 64 == 0) or two or four
// copies of one whole page each (page_size 32 or 16); token rows of 128 or 256 bytes, up to 8 q heads per
// KV head.  Everything else goes to gqa_decode.cu.
//
// Rows of the last tile behind the sequence end are whatever the pool holds: their scores are
// replaced by -inf, and their V rows are zeroed in shared memory by the warp that owns them before
// it reads them (0 x NaN would be NaN).
//
// Work is not pulled from a queue: the tiles of all (sequence, KV head) pairs are cut into one equal
// contiguous range per CTA (stream-K, see segment_at below), which balances ragged batches to one tile,
// needs no cost model, no atomics and almost no plan code, and makes the result bit-reproducible.
//
// Every wait is bounded (the math warps also meet at an mbarrier, not at a hardware barrier); when
// one runs out the CTA records a code in counters[2] (601 producer, 602 math warps waiting for data,
// 603 math warps waiting for each other), raises a flag the other roles poll, and every role leaves.
#include "gqa_decode.cuh"
#include "tb200_async.cuh"

namespace tb200 {
namespace {

#ifndef TB200_DEC_TMA_STAGES16
#define TB200_DEC_TMA_STAGES16 3
#endif
#ifndef TB200_DEC_TMA_BLOCKS16
#define TB200_DEC_TMA_BLOCKS16 2
#endif
#ifndef TB200_DEC_TMA_STAGES8
#define TB200_DEC_TMA_STAGES8 3
#endif
#ifndef TB200_DEC_TMA_BLOCKS8
#define TB200_DEC_TMA_BLOCKS8 3
#endif

constexpr int kTmaThreads = kThreads + 32;   // 4 math warps + the producer warp
constexpr int kItemSlots = 2;                // q rows of the segments the producer may post ahead
constexpr int kMathBarrier = 1;              // named barrier of the 128 math threads (plan only: nothing can give up there)

template <int D, bool FP8>
struct TmaCfg {
  static constexpr int kEsize = FP8 ? 1 : 2;
  static constexpr int kRowBytes = D * kEsize;               // 128 or 256
  static constexpr int kPanels = kRowBytes / 128;            // 128-byte swizzled panels per row
  static constexpr int kPanelElems = 128 / kEsize;
  static constexpr int kPanelBytes = kTile * 128;
  static constexpr int kTensorBytes = kPanels * kPanelBytes; // K (or V) of one tile
  static constexpr int kStageBytes = 2 * kTensorBytes;
  static constexpr int kStages = FP8 ? TB200_DEC_TMA_STAGES8 : TB200_DEC_TMA_STAGES16;
  static constexpr int kBlocks = FP8 ? TB200_DEC_TMA_BLOCKS8 : TB200_DEC_TMA_BLOCKS16;
  static constexpr int kQSlotBytes = 8 * D * 2;              // up to 8 q heads, 16-bit
  static constexpr int kHalf = D / 2;                        // head dims merged per pass
  static constexpr int kMergeStride = kHalf + 4;             // fp32 words per head in the merge area
  static constexpr int kMergeBytes = kWarps * 8 * kMergeStride * 4;
  static constexpr int kMlBytes = kWarps * 8 * 2 * 4;
  // offsets from the 1024-byte aligned base
  static constexpr int ring = 0;
  static constexpr int qslots = ring + kStages * kStageBytes;
  static constexpr int merge = qslots + kItemSlots * kQSlotBytes;
  static constexpr int ml = merge + kMergeBytes;
  static constexpr int scales = ml + kMlBytes;               // [kStages][4 copies][K, V] fp32 (FP8 only)
  static constexpr int bars = scales + 256;                   // full[kStages], empty[kStages], item_full[2], item_empty[2], math
  static constexpr int misc = bars + 8 * (2 * kStages + 2 * kItemSlots + 1);  // 16 ints
  static constexpr int plan = misc + 64;                     // s_prefix [batch + 1], s_lens [batch]
  static_assert(kRowBytes == 128 || kRowBytes == 256, "token rows must be one or two 128-byte panels");
  static_assert(kStages * 8 * 4 <= 256, "scale slots");
};

template <int D, bool FP8>
size_t tma_smem_bytes(int batch) {
  return size_t(TmaCfg<D, FP8>::plan) + size_t(2 * batch + 1) * 4 + 1024;   // + alignment slack
}

// ---- work partition (stream-K) ---------------------------------------------------------------
// A unit is one 64-token tile of one (sequence, KV head, head block) "lane"; units are numbered lane by
// lane (sequence-major), tile by tile.  The T units are cut into equal contiguous ranges, one per CTA
// (range k belongs to CTA k % grid; there is more than one per CTA only when a fixed run length is asked
// for): every CTA gets the same number of tiles to within one, whatever the lengths are, and no CTA ever
// asks a global counter for work.  A range cuts a lane into "segments": a segment that is a whole lane
// writes the output directly; the segments of a lane that several ranges share leave partial (O, max, sum)
// in a slot of their range (2 slots per range: its first segment and its last are the only ones that can
// be partial) and the last one to finish merges them, as in gqa_decode.cu.  The partition is a pure
// function of the lengths, so the producer warp and the math warps walk it independently, and the result
// is bit-reproducible.
struct Segment {
  int b, hk, hbi, rem, len;
  int tile0, tile1;          // tiles of the lane this segment covers
  int n_runs, first_range;   // ranges that share the lane, and the first of them
  int slot;                  // partial-result slot of this segment
  int lane;                  // b * lanes + rem: the lane's ticket
  unsigned lane_start;       // first unit of the lane
  unsigned next;             // first unit behind the segment
};
__device__ __forceinline__ Segment segment_at(const DecodeParams& p, unsigned u, unsigned range_begin, unsigned range_end,
                                              int range, unsigned per, const int* s_prefix, const int* s_lens,
                                              int lanes) {
  Segment g;
  int lo = 0, hi = p.batch - 1;  // the sequence that holds unit u: largest b with lanes * prefix[b] <= u
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (unsigned(s_prefix[mid]) * unsigned(lanes) <= u) lo = mid; else hi = mid - 1;
  }
  g.b = lo;
  g.len = max(s_lens[lo], 0);
  const unsigned tiles_b = unsigned(s_prefix[lo + 1] - s_prefix[lo]);
  const unsigned local = u - unsigned(s_prefix[lo]) * unsigned(lanes);
  g.rem = int(local / tiles_b);
  const unsigned t = local - unsigned(g.rem) * tiles_b;
  g.hk = g.rem / p.n_hb;
  g.hbi = g.rem - g.hk * p.n_hb;
  g.lane = lo * lanes + g.rem;
  g.lane_start = u - t;
  const unsigned lane_end = g.lane_start + tiles_b;
  g.next = min(range_end, lane_end);
  g.tile0 = int(t);
  g.tile1 = int(t + (g.next - u));
  g.first_range = int(g.lane_start / per);
  g.n_runs = int((lane_end - 1) / per) - g.first_range + 1;
  g.slot = 2 * range + (u == range_begin ? 0 : 1);
  return g;
}
// Slot of the segment that range k contributes to the lane starting at lane_start: the range's first
// segment when the lane holds the range's first unit, else its last.
__device__ __forceinline__ int segment_slot(int k, unsigned per, unsigned lane_start) {
  return 2 * k + (unsigned(k) * per >= lane_start ? 0 : 1);
}

// Exclusive scan of the tile counts: s_prefix[0..batch], and the lengths in s_lens.  Called by the 128 math
// threads; `sync` is a barrier over exactly those.
template <typename Sync>
__device__ __forceinline__ void tile_prefix_plan(const DecodeParams& p, int tid, int* s_prefix, int* s_lens,
                                                 int* s_warp_sums, int* s_ragged, Sync sync) {
  const int lane = tid & 31, warp = tid >> 5;
  const int per = (p.batch + kThreads - 1) / kThreads;
  const int b0 = tid * per;
  const int first_len = p.lens ? p.lens[0] : p.uniform_len;
  const int first_tiles = (max(first_len, 0) + kTile - 1) / kTile;
  int sum = 0;
  bool ragged = false;             // some sequence has another number of tiles than sequence 0
  for (int i = 0; i < per; ++i) {
    const int b = b0 + i;
    if (b < p.batch) {
      const int len = p.lens ? p.lens[b] : p.uniform_len;
      s_lens[b] = len;
      const int t = (max(len, 0) + kTile - 1) / kTile;
      ragged |= t != first_tiles;
      sum += t;
    }
  }
  ragged = __any_sync(0xffffffffu, ragged);
  if (lane == 0) s_ragged[warp] = ragged ? 1 : 0;
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) s_warp_sums[warp] = incl;
  sync();
  int run = incl - sum;
  for (int w = 0; w < warp; ++w) run += s_warp_sums[w];
  for (int i = 0; i < per; ++i) {
    const int b = b0 + i;
    if (b < p.batch) {
      s_prefix[b] = run;
      run += (max(s_lens[b], 0) + kTile - 1) / kTile;
    }
    if (b == p.batch - 1) s_prefix[p.batch] = run;
  }
}

// T : MMA element type (bf16 or f16; f16 for FP8 caches, q is converted).  TO : output type.
template <int D, bool FP8, typename T, typename TO>
__global__ void __launch_bounds__(kTmaThreads, TmaCfg<D, FP8>::kBlocks)
gqa_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      DecodeParams p) {
  using C = TmaCfg<D, FP8>;
  constexpr int NT = 1;
  constexpr int kKSteps = D / 16;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::bars);
  auto bar_full = [&](int s) { return smem_u32(bars + s); };
  auto bar_empty = [&](int s) { return smem_u32(bars + C::kStages + s); };
  auto bar_item_full = [&](int s) { return smem_u32(bars + 2 * C::kStages + s); };
  auto bar_item_empty = [&](int s) { return smem_u32(bars + 2 * C::kStages + kItemSlots + s); };
  const uint32_t bar_math = smem_u32(bars + 2 * C::kStages + 2 * kItemSlots);
  int* s_misc = reinterpret_cast<int*>(smem + C::misc);    // [0] abort, [1] ticket, [2..5] warp sums, [8..11] ragged flags
  volatile int* s_abort = s_misc;
  int* s_prefix = reinterpret_cast<int*>(smem + C::plan);  // [batch + 1]
  int* s_lens = s_prefix + p.batch + 1;                    // [batch]
  float* s_scales = reinterpret_cast<float*>(smem + C::scales);
  int* status = p.counters + 2;

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(bar_full(s), 1);
      mbar_init(bar_empty(s), kWarps);
    }
    for (int s = 0; s < kItemSlots; ++s) {
      mbar_init(bar_item_full(s), 1);
      mbar_init(bar_item_empty(s), kThreads);   // every math thread arrives: an arrival orders only its own reads
    }
    mbar_init(bar_math, kThreads);   // every math thread arrives (see math_sync)
    s_misc[0] = 0;
    mbar_fence_init();
  }
  const int step = p.world > 1 ? *reinterpret_cast<volatile int*>(p.step_counter) + 1 : 0;
  const int parity = step & 1;
  const int lanes_per_run = p.heads_kv * p.n_hb;

  if (warp < kWarps)
    tile_prefix_plan(p, tid, s_prefix, s_lens, s_misc + 2, s_misc + 8, [] { named_barrier(kMathBarrier, kThreads); });
  __syncthreads();
  const unsigned total_units = unsigned(s_prefix[p.batch]) * unsigned(lanes_per_run);
  // Units per range.  Default: an equal share per CTA, lanes cut wherever the share ends (a cut costs a
  // partial result, a ticket and a merge: about 8 us of a CTA's time on B200).  A batch whose sequences all
  // have the same length is cut at aligned places instead - whole lanes, or lanes halved k times until the
  // ranges fill the CTAs - when that wastes little: the CTAs then walk the KV heads of the same tokens in
  // step, whole lanes need no merge at all, and on uniform batches of 4k-16k tokens it measured 5-30 %
  // faster than the balanced cut.  Long lanes (>= 256 tiles per CTA) keep the balanced cut: there the
  // idle CTAs of an aligned cut cost more than the merges.
  unsigned per = max((total_units + gridDim.x - 1) / gridDim.x, 1u);
  if (p.force_chunk > 0) {
    per = unsigned(p.force_chunk);
  } else if (!(s_misc[8] | s_misc[9] | s_misc[10] | s_misc[11]) && total_units > 0 && per < 256u) {
    const unsigned L = unsigned(s_prefix[1]);                         // tiles per lane
    const unsigned lanes_total = unsigned(p.batch) * unsigned(lanes_per_run);
    // Runs shorter than kMinRun tiles are not worth their cut: measured on one sequence with 4 KV heads
    // (graph-replayed launches), 1k tokens take 13.7 us uncut against 17.4 us in 16 runs per lane, 8k tokens
    // 19.4 us in runs of 16 tiles against 24-26 us in runs of 4.
    constexpr unsigned kMinRun = 16;
    unsigned k = 1;
    while (k < 32u && 5u * lanes_total * k < 4u * gridDim.x && L % (2u * k) == 0u && L / (2u * k) >= kMinRun) k *= 2u;
    const unsigned ranges = lanes_total * k, waves = (ranges + gridDim.x - 1) / gridDim.x;
    if (4u * ranges >= 3u * waves * gridDim.x || k == 32u || L / (2u * k) < kMinRun) per = L / k;
  }
  // never so small that the ranges outnumber the partial-result slots of the workspace (2 per range)
  per = max(max(per, 1u), (2u * total_units + unsigned(p.max_items) - 1) / unsigned(p.max_items));
  const int n_ranges = int((total_units + per - 1) / per);
  const long long limit = p.wait_cycles;

  if (warp == kWarps) {
    // ================= producer: q rows and K/V tiles of this CTA's segments =================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    int stage = 0;
    uint32_t stage_par = 0;
    bool alive = true;
    int round = 0;
    for (int range = blockIdx.x; alive && range < n_ranges; range += gridDim.x) {
     const unsigned range_begin = unsigned(range) * per, range_end = min(range_begin + per, total_units);
     for (unsigned u = range_begin; alive && u < range_end; ++round) {
      const int slot = round & 1;
      const uint32_t slot_par = (round >> 1) & 1;
      int ok = 1;
      if (lane == 0) ok = mbar_wait_bounded(bar_item_empty(slot), slot_par ^ 1, s_abort, status, 601, limit) ? 1 : 0;
      if (!__shfl_sync(0xffffffffu, ok, 0)) { alive = false; break; }
      const Segment d = segment_at(p, u, range_begin, range_end, range, per, s_prefix, s_lens, lanes_per_run);
      u = d.next;
      const int head0 = d.hk * p.group + d.hbi * p.hb;
      const int n_heads = min(p.hb, p.group - d.hbi * p.hb);
      if (lane == 0) {
        const uint32_t q_bytes = uint32_t(n_heads) * D * 2;
        mbar_expect_tx(bar_item_full(slot), q_bytes);
        bulk_load(sbase + C::qslots + slot * C::kQSlotBytes,
                  reinterpret_cast<const unsigned char*>(p.q) + (size_t(d.b) * p.heads + head0) * D * 2, q_bytes,
                  bar_item_full(slot));
      }
      const int32_t* bt_row = p.bt ? p.bt + size_t(d.b) * p.bt_stride : nullptr;
      const int coord_b = p.bt ? 0 : d.b;
      const int nb = kTile / p.box_rows;    // copies per tile and panel: 1, or 2 / 4 when a tile spans pages of 32 / 16 tokens
      for (int t0 = d.tile0; t0 < d.tile1 && alive; t0 += 32) {
        // 32 tiles per round: lane l reads the table entries (and the scales) of tile t0 + l
        const int t = t0 + lane;
        int tok[4] = {0, 0, 0, 0};            // pool row of each copy of the tile
        float ks[4] = {0.f, 0.f, 0.f, 0.f}, vs[4] = {0.f, 0.f, 0.f, 0.f};   // and, for an e4m3 cache, its page's scales
        if (t < d.tile1) {
          tok[0] = t * kTile;
          if (bt_row) {
            if (nb == 1) {
              const int pg = bt_row[tok[0] / p.page_size];
              tok[0] = pg * p.page_size + tok[0] % p.page_size;
              if constexpr (FP8) {
                ks[0] = p.k_scale[size_t(pg) * p.heads_kv + d.hk];
                vs[0] = p.v_scale[size_t(pg) * p.heads_kv + d.hk];
              }
            } else {
              // one whole page per copy.  The last tile may reach past the sequence's pages: a copy that
              // starts behind the last token re-reads the page of that token (its rows are masked and
              // their V cleared), never a table entry behind the sequence's own.
#pragma unroll
              for (int x = 3; x >= 0; --x) {
                if (x < nb) {
                  const int pg = bt_row[min(t * kTile + x * p.box_rows, d.len - 1) / p.page_size];
                  tok[x] = pg * p.page_size;
                  if constexpr (FP8) {
                    ks[x] = p.k_scale[size_t(pg) * p.heads_kv + d.hk];
                    vs[x] = p.v_scale[size_t(pg) * p.heads_kv + d.hk];
                  }
                }
              }
            }
          }
        }
        const int n = min(32, d.tile1 - t0);
        for (int i = 0; i < n; ++i) {
          int tok_i[4];
          float ks_i[4] = {0.f, 0.f, 0.f, 0.f}, vs_i[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int x = 0; x < 4; ++x) {
            const bool used = x == 0 || nb > 1;            // uniform across the warp
            tok_i[x] = used ? __shfl_sync(0xffffffffu, tok[x], i) : 0;
            if constexpr (FP8) {
              if (used) {
                ks_i[x] = __shfl_sync(0xffffffffu, ks[x], i);
                vs_i[x] = __shfl_sync(0xffffffffu, vs[x], i);
              }
            }
          }
          if (lane == 0) {
            if (mbar_wait_bounded(bar_empty(stage), stage_par ^ 1, s_abort, status, 601, limit)) {
              if constexpr (FP8) {
#pragma unroll
                for (int x = 0; x < 4; ++x) {
                  s_scales[stage * 8 + x * 2] = ks_i[x];
                  s_scales[stage * 8 + x * 2 + 1] = vs_i[x];
                }
              }
              mbar_expect_tx(bar_full(stage), C::kStageBytes);
              const uint32_t dst = sbase + C::ring + stage * C::kStageBytes;
#pragma unroll
              for (int x = 0; x < 4; ++x) {
                if (x < nb) {
                  const uint32_t dx = dst + x * p.box_rows * 128;
#pragma unroll
                  for (int pn = 0; pn < C::kPanels; ++pn)
                    tma_load_4d(dx + pn * C::kPanelBytes, &map_k, bar_full(stage), pn * C::kPanelElems, d.hk, tok_i[x], coord_b);
#pragma unroll
                  for (int pn = 0; pn < C::kPanels; ++pn)
                    tma_load_4d(dx + C::kTensorBytes + pn * C::kPanelBytes, &map_v, bar_full(stage), pn * C::kPanelElems,
                                d.hk, tok_i[x], coord_b);
                }
              }
            } else {
              ok = 0;
            }
          }
          if (!__shfl_sync(0xffffffffu, ok, 0)) { alive = false; break; }
          if (++stage == C::kStages) { stage = 0; stage_par ^= 1; }
        }
      }
     }
    }
  } else {
    // ================= math warps =================
    const int g8 = lane >> 2;  // "groupID" of the mma fragment layouts
    const int t4 = lane & 3;   // "threadID_in_group"
    const float qk_scale = p.softcap > 0.f ? p.sm_scale : p.sm_scale * kLog2e;
    const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;

    // Per-lane ldmatrix offsets inside a swizzled tile.  Row r of a panel is 128 bytes at r * 128 and
    // its 16-byte chunk c sits at (c ^ (r & 7)) * 16.  A k-step (16 elements of a 16-bit cache, 32 of
    // an FP8 one) is two chunks, 2*step and 2*step + 1; the lane's chunk parity and row are fixed, so
    // the four possible values of (2*step) & 7 give four offsets, and the panel is an immediate.
    //   K (both paths) and FP8 V: row = (l&7) + ((l>>3)&1)*8, chunk parity = l>>4
    //   16-bit V (trans):         row = (l&7) + ((l>>4)&1)*8, chunk parity = (l>>3)&1
    uint32_t ka[4], va[4];
    {
      const int x = lane & 7;
      const int row_a = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      const int col_a = lane >> 4;
      const int row_v = FP8 ? row_a : warp * 16 + (lane & 7) + ((lane >> 4) & 1) * 8;
      const int col_v = FP8 ? col_a : (lane >> 3) & 1;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        ka[i] = row_a * 128 + ((i * 32) ^ ((col_a ^ x) << 4));
        va[i] = C::kTensorBytes + row_v * 128 + ((i * 32) ^ ((col_v ^ x) << 4));
      }
    }

    // Barrier of the four math warps with a bounded wait (an mbarrier): a warp that has given up simply
    // never arrives, and the others give up too instead of waiting forever at a hardware barrier.
    // EVERY thread arrives: an arrival releases the arriving thread's own earlier stores, nobody else's.
    // With one arrival per warp (lane 0 behind a __syncwarp) the other lanes' last shared-memory stores
    // before the barrier could still be on their way when another warp, released by the barrier, read them:
    // the 16 head dims a warp writes last into the merge area came out stale (another segment's values) for
    // one (sequence, KV head) in 1-10 % of launches whose CTAs walk many short segments.
    uint32_t math_par = 0;
    bool alive = true;
    auto math_sync = [&]() -> bool {
      mbar_arrive(bar_math);
      const bool ok = mbar_wait_bounded(bar_math, math_par, s_abort, status, 603, limit);
      math_par ^= 1;
      if (!ok) alive = false;
      return ok;
    };

    // ---- split-KV merge, deferred (as in gqa_decode.cu) ---------------------------------------
    struct Pending {
      bool valid;
      int* ticket;
      int n_runs, first_range, b, head0, n_heads;
      unsigned lane_start;
    } pend{false, nullptr, 0, 0, 0, 0, 0, 0u};
    auto resolve_pending = [&]() {
      if (!pend.valid) return;           // uniform across the math warps
      pend.valid = false;
      if (tid == 0) {
        int t;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(t) : "l"(pend.ticket) : "memory");
        s_misc[1] = t;
      }
      if (!math_sync()) return;
      const bool last = s_misc[1] == pend.n_runs - 1;
      if (!math_sync()) return;   // s_misc[1] may be rewritten by the next item's ticket
      if (!last) return;
      // Every thread owns kVec groups of four consecutive head dims (of one head each): 16-byte loads of the
      // partials, one (max, sum) pair and two exponentials per group and run, 16-byte stores of the result.
      constexpr int kVec = (8 * NT * D) / (4 * kThreads);
      float4 acc[kVec];
      float L[kVec], M[kVec];
#pragma unroll
      for (int k = 0; k < kVec; ++k) { acc[k] = make_float4(0.f, 0.f, 0.f, 0.f); L[k] = 0.f; M[k] = kNegFloor; }
      const int n_out = pend.n_heads * D;
#pragma unroll 4   // four runs in flight: a lane cut into 32 runs (one long sequence over all SMs) merges 5 % faster than with two
      for (int r = 0; r < pend.n_runs; ++r) {
        const size_t it2 = size_t(segment_slot(pend.first_range + r, per, pend.lane_start));
        const float* ml = p.part_ml + it2 * p.hb * 2;
        const float* po2 = p.part_o + it2 * p.hb * D;
        float mt[kVec], lt[kVec];
        float4 ot[kVec];
#pragma unroll
        for (int k = 0; k < kVec; ++k) {
          const int idx = (tid + k * kThreads) * 4;
          const bool ok = idx < n_out;
          const int hn = ok ? idx / D : 0;
          mt[k] = ok ? __ldcg(ml + hn * 2) : kNegFloor;
          lt[k] = ok ? __ldcg(ml + hn * 2 + 1) : 0.f;
          ot[k] = ok ? __ldcg(reinterpret_cast<const float4*>(po2 + idx)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int k = 0; k < kVec; ++k) {
          const float mn = fmaxf(M[k], mt[k]);
          const float ea = fast_exp2(M[k] - mn), eb = fast_exp2(mt[k] - mn);
          acc[k].x = acc[k].x * ea + ot[k].x * eb;
          acc[k].y = acc[k].y * ea + ot[k].y * eb;
          acc[k].z = acc[k].z * ea + ot[k].z * eb;
          acc[k].w = acc[k].w * ea + ot[k].w * eb;
          L[k] = L[k] * ea + lt[k] * eb;
          M[k] = mn;
        }
      }
#pragma unroll
      for (int k = 0; k < kVec; ++k) {
        const int idx = (tid + k * kThreads) * 4;
        if (idx < n_out) {
          const int hn = idx / D, d = idx - hn * D;
          const size_t orow = size_t(pend.b) * p.heads + pend.head0 + hn;
          const bool any = L[k] > 0.f;
          emit_out4<TO>(p, parity, orow, d, D,
                        make_float4(any ? acc[k].x / L[k] : 0.f, any ? acc[k].y / L[k] : 0.f,
                                    any ? acc[k].z / L[k] : 0.f, any ? acc[k].w / L[k] : 0.f));
          if (d == 0) emit_lse(p, parity, orow, D, any ? M[k] + log2f(L[k]) : -INFINITY);
        }
      }
      if (tid == 0) *pend.ticket = 0;  // leave the workspace zeroed for the next launch
    };

    int stage = 0;
    uint32_t stage_par = 0;
    int round = 0;
    for (int range = blockIdx.x; alive && range < n_ranges; range += gridDim.x) {
     const unsigned range_begin = unsigned(range) * per, range_end = min(range_begin + per, total_units);
     for (unsigned u = range_begin; alive && u < range_end; ++round) {
      const int slot = round & 1;
      if (!mbar_wait_bounded(bar_item_full(slot), (round >> 1) & 1, s_abort, status, 602, limit)) { alive = false; break; }
      const Segment d = segment_at(p, u, range_begin, range_end, range, per, s_prefix, s_lens, lanes_per_run);
      u = d.next;
      const int b = d.b, hk = d.hk, len = d.len;
      const int n_tiles = d.tile1 - d.tile0;
      const int head0 = hk * p.group + d.hbi * p.hb;
      const int n_heads = min(p.hb, p.group - d.hbi * p.hb);

      // ---- q fragments (B operand of S^T = K Q^T) from the item slot ----------------------------
      uint32_t qf[kKSteps][2];
      {
        const unsigned char* qs = smem + C::qslots + slot * C::kQSlotBytes;
        const bool ok = g8 < n_heads;
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
          if constexpr (!FP8) {
            const uint32_t* qp = reinterpret_cast<const uint32_t*>(qs + (size_t(g8) * D + ks * 16 + t4 * 2) * 2);
            qf[ks][0] = ok ? qp[0] : 0u;
            qf[ks][1] = ok ? qp[4] : 0u;
          } else {
            // k index 2t,2t+1 <-> d = 16ks+4t+{0,1}; k index 2t+8,2t+9 <-> d = 16ks+4t+{2,3}
            float f[4] = {0.f, 0.f, 0.f, 0.f};
            if (ok) {
              const uint2 w = *reinterpret_cast<const uint2*>(qs + (size_t(g8) * D + ks * 16 + t4 * 4) * 2);
              if (p.q_is_bf16) {
                const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w.x);
                const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(&w.y);
                f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(c); f[3] = __high2float(c);
              } else {
                const __half2 a = *reinterpret_cast<const __half2*>(&w.x);
                const __half2 c = *reinterpret_cast<const __half2*>(&w.y);
                f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(c); f[3] = __high2float(c);
              }
            }
            qf[ks][0] = pack2<__half>(f[0], f[1]);
            qf[ks][1] = pack2<__half>(f[2], f[3]);
          }
        }
      }
      mbar_arrive(bar_item_empty(slot));   // id and q rows are in registers (every thread: its own reads)
      resolve_pending();   // ticket / merge of the previous item, while the producer streams this one
      if (!alive) break;

      // ---- running state ----------------------------------------------------------------
      float oacc[kKSteps][4];
      float m_run[2] = {kNegFloor, kNegFloor}, l_run[2] = {0.f, 0.f};
#pragma unroll
      for (int mt = 0; mt < kKSteps; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[mt][e] = 0.f;

      for (int it = 0; it < n_tiles; ++it) {
        if (!mbar_wait_bounded(bar_full(stage), stage_par, s_abort, status, 602, limit)) { alive = false; break; }
        const uint32_t st_base = sbase + C::ring + stage * C::kStageBytes;
        const int tok0 = (d.tile0 + it) * kTile;
        const int tok_a = tok0 + warp * 16 + g8;  // token of c0/c1; c2/c3 is +8
        if (tok0 + kTile > len) {
          // ragged last tile of the sequence: clear this warp's V rows behind the end
          constexpr int kChunks = C::kRowBytes / 16;
          for (int idx = lane; idx < 16 * kChunks; idx += 32) {
            const int row = warp * 16 + idx / kChunks, ch = idx % kChunks;
            if (tok0 + row >= len)
              *reinterpret_cast<uint4*>(smem + C::ring + stage * C::kStageBytes + C::kTensorBytes +
                                        (ch >> 3) * C::kPanelBytes + row * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          // every lane completes its own stores (CTA scope, then towards the async proxy) before the warp goes on:
          // lane 0 alone will hand the stage back to the TMA, and an arrival orders only the arriving thread's stores
          __threadfence_block();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
        }

        // ---- S^T = K Q^T  (16 tokens x 8 heads per warp) ------------------------------------
        float sacc[4] = {0.f, 0.f, 0.f, 0.f}, sacc2[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (!FP8) {
#pragma unroll
          for (int ks = 0; ks < kKSteps; ++ks) {
            uint32_t a[4];
            ldmatrix_x4(a, st_base + (ks >> 2) * C::kPanelBytes + ka[ks & 3]);
            mma_16816<T>((ks & 1) ? sacc2 : sacc, a, qf[ks]);
          }
        } else {
#pragma unroll
          for (int jj = 0; jj < D / 32; ++jj) {
            uint32_t r[4];
            ldmatrix_x4(r, st_base + (jj >> 2) * C::kPanelBytes + ka[jj & 3]);
            uint32_t a0[4] = {e4m3x2_to_f16x2_scaled<0x1404>(r[0]), e4m3x2_to_f16x2_scaled<0x1404>(r[1]),
                              e4m3x2_to_f16x2_scaled<0x3424>(r[0]), e4m3x2_to_f16x2_scaled<0x3424>(r[1])};
            uint32_t a1[4] = {e4m3x2_to_f16x2_scaled<0x1404>(r[2]), e4m3x2_to_f16x2_scaled<0x1404>(r[3]),
                              e4m3x2_to_f16x2_scaled<0x3424>(r[2]), e4m3x2_to_f16x2_scaled<0x3424>(r[3])};
            mma_16816<T>(sacc, a0, qf[2 * jj]);
            mma_16816<T>(sacc2, a1, qf[2 * jj + 1]);
          }
        }

        // ---- scale, softcap, mask, online softmax ----------------------------------------
        // one K scale and one V scale per page; this warp's 16 rows lie in one page (the tile's only one, or
        // with pages of 32 / 16 tokens the tile's copy number warp / 2 or warp)
        float sc = qk_scale, vsc = 1.f;
        if constexpr (FP8) {
          const int copy = (warp * 16) / p.box_rows;
          sc *= s_scales[stage * 8 + copy * 2] * kE4m3Unit;
          vsc = s_scales[stage * 8 + copy * 2 + 1] * kE4m3Unit;
        }
        const bool ok_lo = tok_a < len, ok_hi = tok_a + 8 < len;
        uint32_t pb[2];
        {
          float s0 = (sacc[0] + sacc2[0]) * sc, s1 = (sacc[1] + sacc2[1]) * sc;
          float s2 = (sacc[2] + sacc2[2]) * sc, s3 = (sacc[3] + sacc2[3]) * sc;
          if (p.softcap > 0.f) {
            s0 = apply_softcap(s0, p.softcap, inv_cap) * kLog2e;
            s1 = apply_softcap(s1, p.softcap, inv_cap) * kLog2e;
            s2 = apply_softcap(s2, p.softcap, inv_cap) * kLog2e;
            s3 = apply_softcap(s3, p.softcap, inv_cap) * kLog2e;
          }
          if (!ok_lo) { s0 = -INFINITY; s1 = -INFINITY; }
          if (!ok_hi) { s2 = -INFINITY; s3 = -INFINITY; }
          float mx0 = fmaxf(s0, s2), mx1 = fmaxf(s1, s3);
#pragma unroll
          for (int o = 4; o < 32; o <<= 1) {
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, o));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, o));
          }
          const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
          const float al0 = fast_exp2(m_run[0] - mn0), al1 = fast_exp2(m_run[1] - mn1);
          m_run[0] = mn0; m_run[1] = mn1;
          const float p0 = fast_exp2(s0 - mn0), p1 = fast_exp2(s1 - mn1);
          const float p2 = fast_exp2(s2 - mn0), p3 = fast_exp2(s3 - mn1);
          l_run[0] = l_run[0] * al0 + p0 + p2;
          l_run[1] = l_run[1] * al1 + p1 + p3;
#pragma unroll
          for (int mt = 0; mt < kKSteps; ++mt) {
            oacc[mt][0] *= al0; oacc[mt][1] *= al1;
            oacc[mt][2] *= al0; oacc[mt][3] *= al1;
          }
          // P^T as the B operand: transpose the two 8x8 (token x head) blocks across the warp
          pb[0] = movmatrix_trans(pack2<T>(p0 * vsc, p1 * vsc));
          pb[1] = movmatrix_trans(pack2<T>(p2 * vsc, p3 * vsc));
        }

        // ---- O^T += V^T P^T ------------------------------------------------------------------
        if constexpr (!FP8) {
#pragma unroll
          for (int mt = 0; mt < kKSteps; ++mt) {
            uint32_t a[4];
            ldmatrix_x4_trans(a, st_base + (mt >> 2) * C::kPanelBytes + va[mt & 3]);
            mma_16816<T>(oacc[mt], a, pb);
          }
        } else {
#pragma unroll
          for (int ii = 0; ii < D / 32; ++ii) {
            uint32_t r[4];
            ldmatrix_x4_trans(r, st_base + (ii >> 2) * C::kPanelBytes + va[ii & 3]);
            // register = 2 tokens x 2 dims; bytes (0,2) are dim 2*g8, bytes (1,3) dim 2*g8+1
            uint32_t a0[4] = {e4m3x2_to_f16x2_scaled<0x2404>(r[0]), e4m3x2_to_f16x2_scaled<0x3414>(r[0]),
                              e4m3x2_to_f16x2_scaled<0x2404>(r[1]), e4m3x2_to_f16x2_scaled<0x3414>(r[1])};
            uint32_t a1[4] = {e4m3x2_to_f16x2_scaled<0x2404>(r[2]), e4m3x2_to_f16x2_scaled<0x3414>(r[2]),
                              e4m3x2_to_f16x2_scaled<0x2404>(r[3]), e4m3x2_to_f16x2_scaled<0x3414>(r[3])};
            mma_16816<T>(oacc[2 * ii], a0, pb);
            mma_16816<T>(oacc[2 * ii + 1], a1, pb);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_empty(stage));
        if (++stage == C::kStages) { stage = 0; stage_par ^= 1; }
      }
      if (!alive) break;

      // ---- the 4 warps meet: per-warp (m, l, O^T) -> shared memory, half of the head dims per pass ----
      float* s_o = reinterpret_cast<float*>(smem + C::merge);   // [warp][8][kMergeStride]
      float* s_ml = reinterpret_cast<float*>(smem + C::ml);     // [warp][8][2]
      {
        float l0 = l_run[0], l1 = l_run[1];
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          l0 += __shfl_xor_sync(0xffffffffu, l0, o);
          l1 += __shfl_xor_sync(0xffffffffu, l1, o);
        }
        if (g8 == 0) {
          float* ml = s_ml + (warp * 8 + t4 * 2) * 2;
          ml[0] = m_run[0]; ml[1] = l0; ml[2] = m_run[1]; ml[3] = l1;
        }
      }
      const bool single = (d.n_runs == 1);
      float* po = p.part_o + size_t(d.slot) * p.hb * D;
      float* pml = p.part_ml + size_t(d.slot) * p.hb * 2;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float* so0 = s_o + (warp * 8 + t4 * 2) * C::kMergeStride;
        float* so1 = so0 + C::kMergeStride;
#pragma unroll
        for (int m2 = 0; m2 < kKSteps / 2; ++m2) {
          const int mt = half * (kKSteps / 2) + m2;
          // fragment rows -> head dims: 16-bit path rows g8, g8+8 of the m-tile; FP8 path the
          // ldmatrix on byte pairs interleaves them: rows g8, g8+8 are dims 2*g8, 2*g8+1
          const int d_lo = FP8 ? m2 * 16 + 2 * g8 : m2 * 16 + g8;
          const int d_hi = FP8 ? d_lo + 1 : d_lo + 8;
          so0[d_lo] = oacc[mt][0]; so1[d_lo] = oacc[mt][1];
          so0[d_hi] = oacc[mt][2]; so1[d_hi] = oacc[mt][3];
        }
        if (!math_sync()) break;
        for (int idx = tid; idx < n_heads * C::kHalf; idx += kThreads) {
          const int hn = idx / C::kHalf, dl = idx - hn * C::kHalf;
          const int dd = half * C::kHalf + dl;
          float mw[kWarps], M = kNegFloor;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            mw[w] = s_ml[(w * 8 + hn) * 2];
            M = fmaxf(M, mw[w]);
          }
          float acc = 0.f, L = 0.f;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const float e = fast_exp2(mw[w] - M);
            acc += e * s_o[(w * 8 + hn) * C::kMergeStride + dl];
            L += e * s_ml[(w * 8 + hn) * 2 + 1];
          }
          if (single) {
            const size_t orow = size_t(b) * p.heads + head0 + hn;
            emit_out<TO>(p, parity, orow, dd, D, L > 0.f ? acc / L : 0.f);
            if (dd == 0) emit_lse(p, parity, orow, D, L > 0.f ? M + log2f(L) : -INFINITY);
          } else {
            po[hn * D + dd] = acc;
            if (dd == 0) { pml[hn * 2] = M; pml[hn * 2 + 1] = L; }
          }
        }
        if (!math_sync()) break;   // the area is rewritten by the next pass / item
      }
      if (!alive) break;
      if (!single) {
        // the ticket for this (sequence, KV head, head block) is taken at the start of the next item
        pend.valid = true;
        pend.ticket = p.counters + kCounterWords + d.lane;
        pend.n_runs = d.n_runs;
        pend.first_range = d.first_range;
        pend.lane_start = d.lane_start;
        pend.b = b; pend.head0 = head0; pend.n_heads = n_heads;
      }
     }
    }
    if (alive) resolve_pending();
    // sequences without a single token own no unit: their rows are zero, their LSE -inf
    if (alive) {
      for (int b = blockIdx.x; b < p.batch; b += gridDim.x) {
        if (s_prefix[b + 1] != s_prefix[b]) continue;
        for (int idx = tid; idx < p.heads * D; idx += kThreads) {
          const int h = idx / D, dd = idx - h * D;
          const size_t orow = size_t(b) * p.heads + h;
          emit_out<TO>(p, parity, orow, dd, D, 0.f);
          if (dd == 0) emit_lse(p, parity, orow, D, -INFINITY);
        }
      }
    }

    // ---- the last CTA to leave resets the scheduler counters ------------------------------
    if (p.world > 1) __threadfence_system();   // stores to the other GPUs, out to system scope
    if (alive) math_sync();
    if (tid == 0) {
      __threadfence();
      const int done = atomicAdd(&p.counters[1], 1);
      if (done == int(gridDim.x) - 1) {
        p.counters[0] = 0;
        p.counters[1] = 0;
        __threadfence();
        if (p.world > 1) {
          *p.step_counter = step;
          // ONE system-scope fence, then relaxed flag stores: a release store per peer would be a fence per
          // peer (eight in a row at eight ranks, on the critical path of the step)
          __threadfence_system();
          for (int r = 0; r < p.world; ++r)
            asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p.peer_flag[r]), "r"(step) : "memory");
        }
      }
    }
  }
  if (*s_abort) {
    // give copies still in flight time to land before the shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
}

// ---- host side ------------------------------------------------------------------------------

// [batches, tokens, heads_kv, D] (strides in elements) -> 4-D map (d, head, token, batch) with a box of
// one 128-byte panel x box_rows tokens (64, or one page of 16 or 32), 128B swizzle.  16-bit elements are described as UINT16, e4m3 as UINT8:
// the copy never interprets them.
struct MapKey {
  const void* base;
  int esize, heads_kv, dim, box_rows;
  long long tokens, batches, tok_stride, head_stride, batch_stride;
  bool operator==(const MapKey& o) const {
    return base == o.base && esize == o.esize && heads_kv == o.heads_kv && dim == o.dim && box_rows == o.box_rows &&
           tokens == o.tokens &&
           batches == o.batches && tok_stride == o.tok_stride && head_stride == o.head_stride &&
           batch_stride == o.batch_stride;
  }
};

int encode_kv_map(CUtensorMap* map, const MapKey& k) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return kTmaNotApplicable;
  cuuint64_t dims[4] = {cuuint64_t(k.dim), cuuint64_t(k.heads_kv), cuuint64_t(k.tokens), cuuint64_t(k.batches)};
  cuuint64_t strides[3] = {cuuint64_t(k.head_stride) * k.esize, cuuint64_t(k.tok_stride) * k.esize,
                           cuuint64_t(k.batch_stride) * k.esize};
  cuuint32_t box[4] = {cuuint32_t(128 / k.esize), 1, cuuint32_t(k.box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  // a 256-byte fetch per 128-byte request pays when the neighbouring 128 bytes are the same head's second
  // panel; when a head's row is 128 bytes (e4m3, or 16-bit at head dim 64) they belong to another head,
  // which another CTA reads at another time (measured on an e4m3 cache: ragged batch 133 -> 114 us, 8 x 131072
  // tokens 485 -> 395 us, DRAM traffic 1.29 x -> 1.0 x the algorithmic bytes)
  const CUtensorMapL2promotion promo =
      size_t(k.dim) * k.esize >= 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B;
  CUresult r = enc(map, k.esize == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 4,
                   const_cast<void*>(k.base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return kTmaNotApplicable;   // a layout the copy engine cannot describe: the other kernel serves it
  return TB200_OK;
}

// Encoding a map costs a driver call; decode steps reuse the same pools, so the last few are kept.
int cached_kv_map(CUtensorMap* out, const MapKey& key) {
  constexpr int kSlots = 8;
  struct Slot { MapKey key; CUtensorMap map; bool used; };
  static thread_local Slot cache[kSlots] = {};
  static thread_local int next = 0;
  for (int i = 0; i < kSlots; ++i)
    if (cache[i].used && cache[i].key == key) { *out = cache[i].map; return TB200_OK; }
  CUtensorMap m;
  const int st = encode_kv_map(&m, key);
  if (st != TB200_OK) return st;
  cache[next] = Slot{key, m, true};
  next = (next + 1) % kSlots;
  *out = m;
  return TB200_OK;
}

template <int D, bool FP8, typename T, typename TO>
int launch_tma(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, cudaStream_t stream) {
  auto kern = gqa_decode_tma_kernel<D, FP8, T, TO>;
  const size_t smem = tma_smem_bytes<D, FP8>(p.batch);
  static thread_local size_t configured[64] = {0};
  static thread_local size_t sized_for[64] = {0};
  static thread_local int resident[64] = {0};
  int dev = 0;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return kTmaNotApplicable;
  if (smem > 227 * 1024) return kTmaNotApplicable;
  if (configured[dev] < smem) {
    TB200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  if (sized_for[dev] != smem) {
    int n = 0;
    TB200_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kTmaThreads, smem));
    sized_for[dev] = smem;
    resident[dev] = n < TmaCfg<D, FP8>::kBlocks ? n : TmaCfg<D, FP8>::kBlocks;
  }
  // with fewer resident CTAs than the kernel is tuned for (a very large batch: the plan's tables
  // grow with it) the cp.async kernel is the better choice
  if (resident[dev] < TmaCfg<D, FP8>::kBlocks) return kTmaNotApplicable;
  kern<<<sm_count() * resident[dev], kTmaThreads, smem, stream>>>(mk, mv, p);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}

template <int D, bool FP8, typename T>
int launch_tma_o(const CUtensorMap& mk, const CUtensorMap& mv, const DecodeParams& p, int o_dtype, cudaStream_t s) {
  switch (o_dtype) {
    case TB200_F32: return launch_tma<D, FP8, T, float>(mk, mv, p, s);
    case TB200_BF16: return launch_tma<D, FP8, T, __nv_bfloat16>(mk, mv, p, s);
    case TB200_F16: return launch_tma<D, FP8, T, __half>(mk, mv, p, s);
  }
  return kTmaNotApplicable;
}

}  // namespace

int launch_decode_tma(const DecodeParams& params, int q_dtype, int kv_dtype, int o_dtype, int dim, int nt,
                      long long pool_tokens, cudaStream_t stream) {
  const bool fp8 = kv_dtype == TB200_E4M3;
  const int esize = fp8 ? 1 : 2;
  const int row_bytes = dim * esize;
  if (nt != 1 || (row_bytes != 128 && row_bytes != 256)) return kTmaNotApplicable;
  DecodeParams p = params;
  p.box_rows = kTile;
  if (p.bt && !p.tile_in_page) {
    // pages of 16 or 32 tokens: a tile is 4 or 2 copies of one page each (every math warp's 16 rows still lie
    // in one page, so an e4m3 cache's per-page scales stay one pair per warp and tile)
    if (p.page_size != 16 && p.page_size != 32) return kTmaNotApplicable;
    p.box_rows = p.page_size;
  }
  if (fp8 && !p.bt) return kTmaNotApplicable;              // scales are indexed by page: needs the table
  if (reinterpret_cast<uintptr_t>(p.q) & 15) return kTmaNotApplicable;
  if (p.tok_stride <= 0 || p.head_stride <= 0) return kTmaNotApplicable;
  {
    // the partition counts tiles in 32 bits: bound them by what the cache can hold
    const long long cap = p.bt ? (long long)p.bt_stride * p.page_size
                               : (p.lens ? (p.tok_stride > 0 ? p.batch_stride / p.tok_stride : 0) : (long long)p.uniform_len);
    const long long units = (long long)p.batch * ((cap + kTile - 1) / kTile) * p.heads_kv * p.n_hb;
    if (units >= (1LL << 30)) return kTmaNotApplicable;
  }

  MapKey key{};
  key.esize = esize; key.heads_kv = p.heads_kv; key.dim = dim; key.box_rows = p.box_rows;
  key.tok_stride = p.tok_stride; key.head_stride = p.head_stride;
  if (p.bt) {
    key.tokens = pool_tokens > 0 ? pool_tokens : 0x7fffffffLL;   // unknown pool size: only the table bounds the reads
    key.batches = 1;
    key.batch_stride = p.tok_stride;                              // unused (one batch); any multiple of 16 bytes
  } else {
    if (p.batch_stride <= 0 || p.batch_stride % p.tok_stride != 0) return kTmaNotApplicable;
    key.tokens = p.batch_stride / p.tok_stride;
    key.batches = p.batch;
    key.batch_stride = p.batch_stride;
  }
  if (key.tokens > 0xffffffffLL || (unsigned long long)key.tok_stride * esize >= (1ull << 40) ||
      (unsigned long long)key.batch_stride * esize >= (1ull << 40))
    return kTmaNotApplicable;
  CUtensorMap mk, mv;
  key.base = p.k;
  int st = cached_kv_map(&mk, key);
  if (st != TB200_OK) return st;
  key.base = p.v;
  st = cached_kv_map(&mv, key);
  if (st != TB200_OK) return st;

  if (fp8) {
    return dim == 128 ? launch_tma_o<128, true, __half>(mk, mv, p, o_dtype, stream) : kTmaNotApplicable;
  }
  if (q_dtype == TB200_BF16)
    return dim == 128 ? launch_tma_o<128, false, __nv_bfloat16>(mk, mv, p, o_dtype, stream)
                      : launch_tma_o<64, false, __nv_bfloat16>(mk, mv, p, o_dtype, stream);
  return dim == 128 ? launch_tma_o<128, false, __half>(mk, mv, p, o_dtype, stream)
                    : launch_tma_o<64, false, __half>(mk, mv, p, o_dtype, stream);
}

}  // namespace tb200
