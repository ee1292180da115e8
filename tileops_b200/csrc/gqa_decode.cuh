// Pieces shared by the two single-token GQA decode kernels (gqa_decode.cu: cp.async loads issued
// by the math warps, serves every layout; gqa_decode_tma.cu: a producer warp feeding the math
// warps by TMA, serves caches whose 64-token tiles are contiguous in memory): the launch
// parameters, the workspace layout, the device-side plan and the output stores.
#pragma once

#include "tb200_common.cuh"

namespace tb200 {

constexpr int kTile = 64;          // tokens per shared-memory tile
constexpr int kThreads = 128;      // 4 math warps x 16 tokens
constexpr int kWarps = 4;
constexpr int kMinChunkTiles = 2;  // never cut a sequence into runs shorter than this
#ifndef TB200_DEC_ITEMS_PER_CTA
#define TB200_DEC_ITEMS_PER_CTA 8
#endif
#ifndef TB200_DEC_ITEM_COST16
#define TB200_DEC_ITEM_COST16 2.f
#endif
#ifndef TB200_DEC_SPLIT_COST16
#define TB200_DEC_SPLIT_COST16 3.f
#endif
#ifndef TB200_DEC_ITEM_COST8
#define TB200_DEC_ITEM_COST8 2.f
#endif
#ifndef TB200_DEC_SPLIT_COST8
#define TB200_DEC_SPLIT_COST8 3.f
#endif
constexpr int kItemsPerCta = TB200_DEC_ITEMS_PER_CTA;  // target number of work items per resident CTA
constexpr int kMaxBatch = 4096;
constexpr int kMaxPeers = 8;
constexpr int kCounterWords = 4;   // [0] next item, [1] CTAs done, [2] status, [3] spare; tickets follow

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* lse;
  const int32_t* lens;
  int32_t uniform_len;
  const int32_t* bt;
  int32_t bt_stride;
  const float* k_scale;
  const float* v_scale;
  int batch, heads, heads_kv, group;
  int hb;       // q heads handled by one item (<= 8*NT)
  int n_hb;     // head blocks per KV head
  int page_size;
  int tile_in_page;  // 1 when page_size % 64 == 0: a tile never straddles two pages
  int box_rows;      // TMA kernel: token rows per copy (64, or the page size when a tile spans 2 or 4 pages)
  int64_t tok_stride, head_stride, batch_stride;  // elements
  float sm_scale, softcap;
  int q_is_bf16;
  int target_items;
  int max_items;
  int force_chunk;  // > 0: run length in tiles (the chunk_tiles field of the variant flags)
  int* counters;   // [0] next item, [1] CTAs done, [2] status, [kCounterWords + (b*heads_kv + hk)*n_hb + hb] tickets
  float* part_o;   // [max_items][hb][D]
  float* part_ml;  // [max_items][hb][2]
  // KV-sequence sharding over GPUs (world > 1): the fp32 result and its LSE are stored straight into
  // every rank's exchange buffer over NVLink instead of p.o / p.lse, and the last CTA raises this
  // rank's flag on every rank.  Step number and buffer parity come from a device counter, so the
  // launch can be replayed from a CUDA graph.
  int world;
  float* peer_o[kMaxPeers];     // rank r's buffer base (this rank's slot is selected in the kernel)
  int* peer_flag[kMaxPeers];    // this rank's flag word on rank r
  int* step_counter;            // local; step = *step_counter + 1, written back by the last CTA
  long long slot_floats;        // floats of one rank's slot: batch * heads * (D + 1)
  int rank;
  long long wait_cycles;        // limit of every device-side wait of the TMA kernel (clock64 ticks)
};

__device__ __forceinline__ float apply_softcap(float x, float cap, float inv_cap) {
  return cap * fast_tanh(x * inv_cap);
}

// Final (normalised) output element and LSE of a (sequence, q head).  Single GPU: to p.o / p.lse.
// Sharded over GPUs: the same fp32 value goes to this rank's slot of the current parity in every
// rank's exchange buffer (plain stores through peer-mapped pointers), O at [row][d], LSE behind it.
template <typename TO>
__device__ __forceinline__ void emit_out(const DecodeParams& p, int parity, size_t row, int d, int dim, float val) {
  if (p.world > 1) {
    const size_t off = (size_t(parity) * p.world + p.rank) * size_t(p.slot_floats) + row * dim + d;
    for (int r = 0; r < p.world; ++r) p.peer_o[r][off] = val;
  } else {
    store_out<TO>(reinterpret_cast<TO*>(p.o) + row * dim + d, val);
  }
}
// Four consecutive head dims (d a multiple of 4) of one row.  Sharded: ONE 16-byte store per peer instead of four
// scalar ones - stores to a peer are posted through a short queue, and at 8 ranks the scalar form made the decode
// launch 22 us longer than the local decode - when the slot layout keeps the row 16-byte aligned (it does when
// batch * heads is a multiple of 4; else the scalar form).
template <typename TO>
__device__ __forceinline__ void emit_out4(const DecodeParams& p, int parity, size_t row, int d, int dim, float4 v) {
  if (p.world > 1) {
    const size_t off = (size_t(parity) * p.world + p.rank) * size_t(p.slot_floats) + row * dim + d;
    if ((off & 3) == 0) {
      for (int r = 0; r < p.world; ++r) *reinterpret_cast<float4*>(p.peer_o[r] + off) = v;
    } else {
      for (int r = 0; r < p.world; ++r) {
        float* dst = p.peer_o[r] + off;
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
      }
    }
  } else {
    TO* dst = reinterpret_cast<TO*>(p.o) + row * dim + d;
    store_out<TO>(dst, v.x); store_out<TO>(dst + 1, v.y); store_out<TO>(dst + 2, v.z); store_out<TO>(dst + 3, v.w);
  }
}
__device__ __forceinline__ void emit_lse(const DecodeParams& p, int parity, size_t row, int dim, float val) {
  if (p.world > 1) {
    const size_t off = (size_t(parity) * p.world + p.rank) * size_t(p.slot_floats) +
                       size_t(p.batch) * p.heads * dim + row;
    for (int r = 0; r < p.world; ++r) p.peer_o[r][off] = val;
  } else if (p.lse) {
    p.lse[row] = val;
  }
}

// ---- plan: cut every sequence into runs of tiles (identical in every CTA) -------------------
// The run length is chosen from a short list by a cost model in units of one tile's time:
//   cost(c) = max(W/P, largest run if there are fewer runs than CTAs)
//           + (items per CTA) * kItemCost + (split items per CTA) * kSplitCost
//           + half a run of tail imbalance when CTAs take more than one item
// (W = all tiles, P = CTAs).  Short runs balance ragged batches; long runs avoid the refill of
// the load pipeline, the partial results and the merge; an unsplit sequence costs least per
// item.  Integer sums and maxima are reduced with order-independent atomics, so every CTA
// arrives at the same plan.
//
// Called by 128 threads (tid 0..127) that share `sync` (a barrier over exactly those threads).
// s_scratch: at least 50 ints, free during the call.  On return s_prefix[0..batch] holds the
// exclusive scan of the run counts and s_lens[0..batch) the context lengths; the caller must
// `sync` once more before other threads read them.
template <bool FP8, typename Sync>
__device__ __forceinline__ void decode_plan(const DecodeParams& p, int tid, int* s_scratch, int* s_prefix,
                                            int* s_lens, int* s_warp_sums, Sync sync) {
  const int lane = tid & 31, warp = tid >> 5;
  const int lanes_per_run = p.heads_kv * p.n_hb;
  constexpr int kCand = 16;
  // fixed cost of a work item and of a split item, in units of one tile's time; an FP8 tile is half
  // the bytes of a 16-bit one, so the same microseconds are more tiles
  constexpr float kItemCost = FP8 ? TB200_DEC_ITEM_COST8 : TB200_DEC_ITEM_COST16,
                  kSplitCost = FP8 ? TB200_DEC_SPLIT_COST8 : TB200_DEC_SPLIT_COST16;
  int* s_cand = s_scratch;            // [kCand][3]: items, split items, largest run
  int* s_tot = s_cand + kCand * 3;    // [2]: all tiles, longest sequence in tiles
  if (tid < kCand * 3 + 2) s_cand[tid] = 0;
  sync();
  int local = 0, local_max = 0;
  for (int b = tid; b < p.batch; b += kThreads) {
    const int len = p.lens ? p.lens[b] : p.uniform_len;
    s_lens[b] = len;              // every later use reads this copy (visible after the barrier below)
    const int t = (max(len, 0) + kTile - 1) / kTile;
    local += t;
    local_max = max(local_max, t);
  }
  local = __reduce_add_sync(0xffffffffu, local);
  local_max = __reduce_max_sync(0xffffffffu, local_max);
  if (lane == 0) { atomicAdd(&s_tot[0], local); atomicMax(&s_tot[1], local_max); }
  sync();
  const long long total_tiles = s_tot[0];
  const int max_tiles = max(s_tot[1], 1);
  // the workspace holds batch*lanes + target_items partials: never cut finer than this
  const int c_min = (int)max((long long)kMinChunkTiles,
                             (total_tiles * lanes_per_run + p.target_items - 1) / p.target_items);
  auto cand = [&](int i) {
    // 8, 12, 16, 24, 32, 48, ... , 1024, then "do not split"
    const int c = i == kCand - 1 ? max_tiles : ((i & 1) ? 12 : 8) << (i >> 1);
    return min(max(c, c_min), max(max_tiles, c_min));
  };
  // Thread t scores candidate t % 16 over the sequences b with b % 8 == t / 16: a short rolled loop
  // (the code runs once per CTA straight from a cold instruction cache, so it is kept small) with its
  // three partial results in registers; the 8 threads of a candidate meet in shared memory.
  {
    static_assert(kCand == 16 && kThreads == 128, "the mapping below assumes 16 candidates and 128 threads");
    const int ci = tid & (kCand - 1);
    const int c = cand(ci);
    int it = 0, sp = 0, mx = 0;
#pragma unroll 1
    for (int b = tid >> 4; b < p.batch; b += kThreads / kCand) {
      const int len = s_lens[b];
      const int t = (max(len, 0) + kTile - 1) / kTile;
      const int n = max(1, (t + c - 1) / c);
      it += n;
      sp += n > 1 ? n : 0;
      mx = max(mx, (t + n - 1) / n);
    }
    // lanes l and l + 16 hold the same candidate
    it += __shfl_xor_sync(0xffffffffu, it, 16);
    sp += __shfl_xor_sync(0xffffffffu, sp, 16);
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
    if (lane < kCand) {
      atomicAdd(&s_cand[ci * 3], it);
      atomicAdd(&s_cand[ci * 3 + 1], sp);
      atomicMax(&s_cand[ci * 3 + 2], mx);
    }
  }
  sync();
  int chunk = cand(kCand - 1);
  if (p.force_chunk > 0) {
    chunk = max(p.force_chunk, c_min);
  } else {
    const float P = float(gridDim.x);
    const float w_per_cta = float(total_tiles) * lanes_per_run / P;
    float best = 3.0e38f;
    for (int i = 0; i < kCand; ++i) {
      const float k = float(s_cand[i * 3]) * lanes_per_run / P;
      const float ks = float(s_cand[i * 3 + 1]) * lanes_per_run / P;
      const float big = float(s_cand[i * 3 + 2]);
      const float cost = fmaxf(w_per_cta, k <= 1.f ? big : 0.f) + k * kItemCost + ks * kSplitCost +
                         (k > 1.f ? 0.5f * big : 0.f);
      if (cost <= best) { best = cost; chunk = cand(i); }   // ties go to the longer run
    }
  }
  sync();   // s_cand may live in memory the caller reuses

  const int per = (p.batch + kThreads - 1) / kThreads;
  const int b0 = tid * per;
  int sum = 0;
  for (int i = 0; i < per; ++i) {
    int b = b0 + i;
    if (b < p.batch) {
      int len = s_lens[b];
      int tiles = (max(len, 0) + kTile - 1) / kTile;
      sum += max(1, (tiles + chunk - 1) / chunk);
    }
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  if (lane == 31) s_warp_sums[warp] = incl;
  sync();
  int base = 0;
  for (int w = 0; w < warp; ++w) base += s_warp_sums[w];
  int run = base + incl - sum;
  for (int i = 0; i < per; ++i) {
    int b = b0 + i;
    if (b < p.batch) {
      s_prefix[b] = run;
      int len = s_lens[b];
      int tiles = (max(len, 0) + kTile - 1) / kTile;
      run += max(1, (tiles + chunk - 1) / chunk);
    }
    if (b == p.batch - 1) s_prefix[p.batch] = run;
  }
}

// What a work item covers, derived from its id and the plan in shared memory.
struct ItemDesc {
  int b, hk, hbi, rem;
  int len, n_runs, first_run;
  int tile0, tile1;
};
__device__ __forceinline__ ItemDesc decode_item(const DecodeParams& p, int item, const int* s_prefix,
                                                const int* s_lens) {
  ItemDesc d;
  const int lanes_per_run = p.heads_kv * p.n_hb;
  const int run = item / lanes_per_run;
  d.rem = item - run * lanes_per_run;
  d.hk = d.rem / p.n_hb;
  d.hbi = d.rem - d.hk * p.n_hb;
  int lo = 0, hi = p.batch - 1;  // largest b with s_prefix[b] <= run
  while (lo < hi) {
    int mid = (lo + hi + 1) >> 1;
    if (s_prefix[mid] <= run) lo = mid; else hi = mid - 1;
  }
  d.b = lo;
  d.len = max(s_lens[lo], 0);
  const int tiles_b = (d.len + kTile - 1) / kTile;
  d.first_run = s_prefix[lo];
  d.n_runs = s_prefix[lo + 1] - d.first_run;
  const int j = run - d.first_run;
  const int run_tiles = (tiles_b + d.n_runs - 1) / d.n_runs;
  d.tile0 = min(j * run_tiles, tiles_b);
  d.tile1 = min(d.tile0 + run_tiles, tiles_b);
  return d;
}

// ---- host side ------------------------------------------------------------------------------
struct Layout {
  size_t counters_bytes, part_o_bytes, part_ml_bytes, total;
  int hb, n_hb, nt, target_items, max_items;
};

// The workspace layout depends only on (batch, heads, heads_kv, dim): every kernel variant uses
// the same one, so a caller sizes it once.
inline Layout make_layout(int batch, int heads, int heads_kv, int dim) {
  Layout L{};
  const int group = heads / heads_kv;
  L.hb = group < 16 ? group : 16;
  L.nt = L.hb <= 8 ? 1 : 2;
  L.n_hb = (group + L.hb - 1) / L.hb;
  L.target_items = sm_count() * 3 * kItemsPerCta;  // independent of the cache dtype
  L.max_items = batch * heads_kv * L.n_hb + L.target_items;
  auto up = [](size_t x) { return (x + 255) & ~size_t(255); };
  L.counters_bytes = up(size_t(kCounterWords + size_t(batch) * heads_kv * L.n_hb) * 4);
  L.part_o_bytes = up(size_t(L.max_items) * L.hb * dim * 4);
  L.part_ml_bytes = up(size_t(L.max_items) * L.hb * 2 * 4);
  L.total = L.counters_bytes + L.part_o_bytes + L.part_ml_bytes;
  return L;
}

// Variant flags of tb200_gqa_decode (see the header): which instantiation serves a call.
struct DecodeVariant {
  int wide;        // -1 library's choice, 0 off, 1 on
  int fp8_mma;     // e4m3 tensor-core path
  int no_tma;      // keep the cp.async kernel even where the TMA kernel applies
  int chunk_tiles; // > 0: fixed run length
};
inline DecodeVariant parse_variant(int flags) {
  DecodeVariant v{};
  v.wide = (flags & TB200_DECODE_WIDE_ON) ? 1 : (flags & TB200_DECODE_WIDE_OFF) ? 0 : -1;
  v.fp8_mma = (flags & TB200_DECODE_FP8_MMA) ? 1 : 0;
  v.no_tma = (flags & TB200_DECODE_NO_TMA) ? 1 : 0;
  v.chunk_tiles = (flags >> TB200_DECODE_CHUNK_TILES_SHIFT) & 0xFFFF;
  return v;
}

// Defined in gqa_decode_tma.cu.  Returns TB200_OK after launching, a negative value when the TMA
// kernel does not serve this call (the caller then launches the cp.async kernel), or an error.
constexpr int kTmaNotApplicable = -1;
int launch_decode_tma(const DecodeParams& p, int q_dtype, int kv_dtype, int o_dtype, int dim, int nt,
                      long long pool_tokens, cudaStream_t stream);

}  // namespace tb200
