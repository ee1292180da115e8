// Single-token GQA decode over a paged or contiguous KV cache, sm_100a.
//
// Role in the reference: replaces GQADecodeKernel and GQADecodePagedKernel
// (src/tileops/kernels/attention/gqa_decode.py:23-306, gqa_decode_paged.py:44-395 in
// tile-ai/TileOPs), including their split-KV combine grid, in ONE launch and without the
// reference's per-call host synchronisation on real_seqlen_kv.max().
//
// The op is HBM bound: every K and V byte is read exactly once.  Design:
//   * work item = (sequence, KV head, contiguous run of 64-token tiles); every CTA derives the
//     same plan from real_seqlen_kv on the device: a small cost model scores 16 candidate run
//     lengths (busiest CTA's tiles + per-item + per-split merge cost) and takes the cheapest;
//     CTAs pull items from an atomic counter (no host sync, no idle tail);
//   * K/V rows are gathered through the block table with 16-byte cp.async into a 3-stage
//     shared-memory ring (rows padded by 16 B so that ldmatrix is bank-conflict free);
//   * tokens sit on the MMA M dimension and the q-head group on N=8
//     (S^T = K Q^T, O^T = V^T P^T, mma.sync.m16n8k16), so no tensor-core row is padding;
//   * each of the 4 warps owns 16 tokens of a tile and keeps its own running max/sum
//     (register + shuffle reductions); the warps meet once per item;
//   * FP8-e4m3 caches are converted to f16 in registers between ldmatrix and mma
//     (cvt.rn.f16x2.e4m3x2), the per-(page, KV head) scales are applied to the fp32 scores
//     (K) and to P (V);
//   * partial (O, max, sum) of an item go to a workspace in fp32; the CTA that finishes a
//     (sequence, KV head) last merges them (acq_rel atomic ticket taken after the next
//     item's loads are issued; nobody waits).
#include "gqa_decode.cuh"

namespace tb200 {
namespace {

#ifndef TB200_DEC_DEFER
#define TB200_DEC_DEFER 1
#endif
#ifndef TB200_DEC_STAGES16
#define TB200_DEC_STAGES16 3
#endif
#ifndef TB200_DEC_BLOCKS16
#define TB200_DEC_BLOCKS16 2
#endif
// FP8 caches: 4 CTAs per SM with a 3-stage ring (at most 128 registers) measured 2-6 % faster on
// ragged and long-context batches than 3 CTAs with 4 stages, and the same on uniform 4k contexts.
// Cross-item prefetch (off: measured 1-6 % SLOWER on B200): while the last tiles of an item are
// computed (no loads of this item are left to issue), the first tiles of the CTA's NEXT item are
// requested into L2, so that the next item's pipeline fill hits L2.  The extra code and live
// registers in the tile loop cost more than the shorter fill saves.
#ifndef TB200_DEC_PREFETCH_NEXT
#define TB200_DEC_PREFETCH_NEXT 0
#endif
#ifndef TB200_DEC_STAGES8
#define TB200_DEC_STAGES8 3
#endif
#ifndef TB200_DEC_BLOCKS8
#define TB200_DEC_BLOCKS8 4
#endif

// WIDE (16-bit caches, up to 8 q heads per KV head): 3 CTAs per SM with a 2-stage ring instead of 2
// CTAs with 3 stages.  Measured on B200: +7.5 % on 131k-token contexts (6.5 TB/s, the copy peak),
// -1 % on ragged 0.5k-8k contexts, -12 % on short uniform batches, so the host picks it only where
// every sequence may be long.
template <int D, bool FP8, bool WIDE = false>
struct Cfg {
  static constexpr int kEsize = FP8 ? 1 : 2;
  static constexpr int kRowBytes = D * kEsize;
  static constexpr int kRowStride = kRowBytes + 16;
  static constexpr int kChunksPerRow = kRowBytes / 16;
  static constexpr int kTileBytes = kTile * kRowStride;
  static constexpr int kStageBytes = 2 * kTileBytes + (FP8 ? 2 * kTile * 4 : 0);
  static constexpr int kStages = FP8 ? TB200_DEC_STAGES8 : (WIDE ? 2 : TB200_DEC_STAGES16);
  static constexpr int kOStride = D + 4;  // fp32 words per head in the cross-warp merge area
};

// Resident CTAs per SM the kernel is compiled for (it bounds the registers per thread): the FP8
// kernel for up to 8 q heads per KV head fits 128 registers, the 16-head one does not.
__host__ __device__ constexpr int min_blocks(bool fp8, int nt, bool wide = false) {
  return fp8 ? (nt == 1 ? TB200_DEC_BLOCKS8 : 3) : (wide ? 3 : TB200_DEC_BLOCKS16);
}

template <int D, bool FP8, bool WIDE = false>
size_t smem_bytes(int batch, int nt) {
  using C = Cfg<D, FP8, WIDE>;
  size_t ring = size_t(C::kStages) * C::kStageBytes;
  size_t merge = size_t(kWarps) * (8 * nt) * (C::kOStride + 2) * 4;
  size_t a = ring > merge ? ring : merge;
  return a + size_t(2 * batch + 1) * 4 + 128;   // run-count prefix [batch + 1] and the lengths [batch]
}

// T  : MMA element type (bf16 or f16).  For FP8 caches T is f16 and q is converted.
// TO : output element type.
// F8M: FP8 cache consumed by e4m3 tensor-core MMAs (m16n8k32) with no expansion at all.  K and V
//      bytes go from ldmatrix straight into the MMA; q and P, which are not e4m3 numbers, enter as
//      the sum of two e4m3 numbers (hi + lo, about 8 significant bits, what bf16 carries), so
//      S^T = K q_hi^T + K q_lo^T (two MMAs per 32 dims) and O^T += [V^T V^T] [P_hi; P_lo] (hi and
//      lo stacked on the k axis of one MMA).  Needs one scale per tile and tensor: tiles that lie
//      inside one page (page_size a multiple of 64); other layouts use the f16 expansion path.
template <int D, bool FP8, typename T, int NT, typename TO, bool F8M = false, bool WIDE = false>
__global__ void __launch_bounds__(kThreads, min_blocks(FP8, NT, WIDE)) gqa_decode_kernel(DecodeParams p) {
  using C = Cfg<D, FP8, WIDE>;
  constexpr int kKSteps = D / 16;  // MMAs per 16 tokens for S^T, and m-tiles of O^T
  extern __shared__ __align__(128) unsigned char smem[];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int g8 = lane >> 2;  // "groupID" of the mma fragment layouts
  const int t4 = lane & 3;   // "threadID_in_group"

  unsigned char* ring = smem;
  constexpr size_t kRing = size_t(C::kStages) * C::kStageBytes;
  constexpr size_t kMerge = size_t(kWarps) * (8 * NT) * (C::kOStride + 2) * 4;
  constexpr size_t kArea = kRing > kMerge ? kRing : kMerge;
  int* s_prefix = reinterpret_cast<int*>(smem + kArea);  // [batch + 1] run counts, exclusive scan
  int* s_lens = s_prefix + p.batch + 1;                   // [batch] context lengths (one global read per CTA)
  int* s_misc = s_lens + p.batch;                         // [1] ticket, [2..5] plan scratch, [6],[7] item ids

  // id of this CTA's first work item: requested now, so that the round trip of the atomic runs
  // under the plan computation; it is stored to shared memory after the plan
  int first_item_id = 0;
  if (tid == 0) first_item_id = atomicAdd(&p.counters[0], 1);
  // sharded over GPUs: number of this step (every CTA reads the same value: the counter is advanced
  // by the last CTA of a launch) and the half of the exchange buffers it uses
  const int step = p.world > 1 ? *reinterpret_cast<volatile int*>(p.step_counter) + 1 : 0;
  const int parity = step & 1;

  const int lanes_per_run = p.heads_kv * p.n_hb;

  // ---- plan: cut every sequence into runs of tiles (identical in every CTA); its scratch lives in the
  // ring, which is not in use yet
  decode_plan<FP8>(p, tid, reinterpret_cast<int*>(smem), s_prefix, s_lens, s_misc + 2, [] { __syncthreads(); });
  __syncthreads();
  const int total_items = s_prefix[p.batch] * lanes_per_run;

  const float qk_scale = p.softcap > 0.f ? p.sm_scale : p.sm_scale * kLog2e;
  const float inv_cap = p.softcap > 0.f ? 1.f / p.softcap : 0.f;

  // per-lane ldmatrix offsets (bytes within a tile, before the k/d step is added)
  //   K (both paths) and FP8 V: row = (l&7) + ((l>>3)&1)*8, 16-byte column block = l>>4
  //   16-bit V (trans):         row = (l&7) + ((l>>4)&1)*8, 16-byte column block = (l>>3)&1
  const int ld_row_a = (lane & 7) + ((lane >> 3) & 1) * 8;
  const int ld_col_a = lane >> 4;
  const int ld_row_v = FP8 ? ld_row_a : (lane & 7) + ((lane >> 4) & 1) * 8;
  const int ld_col_v = FP8 ? ld_col_a : (lane >> 3) & 1;
  const uint32_t ring_u32 = smem_u32(ring);
  const uint32_t k_lane_off = (warp * 16 + ld_row_a) * C::kRowStride + ld_col_a * 16;
  const uint32_t v_lane_off = C::kTileBytes + (warp * 16 + ld_row_v) * C::kRowStride + ld_col_v * 16;

  // ---- split-KV merge, deferred -----------------------------------------------------------
  // A finished run leaves its partial (O, max, sum) in the workspace.  Whoever finishes a
  // (sequence, KV head, head block) last merges all of its runs: thread 0 publishes this CTA's
  // partial (the CTA barrier hands every thread's stores to thread 0, whose release is cumulative
  // and makes them visible device-wide) and takes a ticket.  The atomic costs a round trip to L2,
  // so it runs when the NEXT item's first tiles are already in flight.
  struct Pending {
    bool valid;
    int* ticket;
    int n_runs, first_item, b, head0, n_heads;
  } pend{false, nullptr, 0, 0, 0, 0, 0};
  auto resolve_pending = [&]() {
    if (!pend.valid) return;           // uniform across the CTA
    pend.valid = false;
    if (tid == 0) {
      // release (publishes the partial) + acquire (sees the other runs' partials) in one
      // device-scope atomic; a sequentially consistent __threadfence() would also wait for this
      // thread's loads in flight
      int t;
      asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(t) : "l"(pend.ticket) : "memory");
      s_misc[1] = t;
    }
    __syncthreads();
    if (s_misc[1] != pend.n_runs - 1) return;
    // One pass over the runs with a running maximum.  Each thread owns kOut outputs and issues
    // the loads of a run for all of them before using any, so a merge costs about one memory
    // round trip per run instead of one per run and output.
    constexpr int kOut = (8 * NT * D) / kThreads;
    float acc[kOut], L[kOut], M[kOut];
#pragma unroll
    for (int k = 0; k < kOut; ++k) { acc[k] = 0.f; L[k] = 0.f; M[k] = kNegFloor; }
    const int n_out = pend.n_heads * D;
#pragma unroll 2
    for (int r = 0; r < pend.n_runs; ++r) {
      const size_t it2 = size_t(pend.first_item) + size_t(r) * lanes_per_run;
      const float* ml = p.part_ml + it2 * p.hb * 2;
      const float* po2 = p.part_o + it2 * p.hb * D;
      float mt[kOut], lt[kOut], ot[kOut];
#pragma unroll
      for (int k = 0; k < kOut; ++k) {
        const int idx = tid + k * kThreads;
        const bool ok = idx < n_out;
        const int hn = ok ? idx / D : 0;
        mt[k] = ok ? __ldcg(ml + hn * 2) : kNegFloor;
        lt[k] = ok ? __ldcg(ml + hn * 2 + 1) : 0.f;
        ot[k] = ok ? __ldcg(po2 + idx) : 0.f;     // part_o row is [hn][d] = idx
      }
#pragma unroll
      for (int k = 0; k < kOut; ++k) {
        const float mn = fmaxf(M[k], mt[k]);
        const float ea = fast_exp2(M[k] - mn), eb = fast_exp2(mt[k] - mn);
        acc[k] = acc[k] * ea + ot[k] * eb;
        L[k] = L[k] * ea + lt[k] * eb;
        M[k] = mn;
      }
    }
#pragma unroll
    for (int k = 0; k < kOut; ++k) {
      const int idx = tid + k * kThreads;
      if (idx < n_out) {
        const int hn = idx / D, d = idx - hn * D;
        const size_t orow = size_t(pend.b) * p.heads + pend.head0 + hn;
        emit_out<TO>(p, parity, orow, d, D, L[k] > 0.f ? acc[k] / L[k] : 0.f);
        if (d == 0) emit_lse(p, parity, orow, D, L[k] > 0.f ? M[k] + log2f(L[k]) : -INFINITY);
      }
    }
    if (tid == 0) *pend.ticket = 0;  // leave the workspace zeroed for the next launch
  };

  // Item ids are fetched one item ahead (two alternating slots), so the round trip of the
  // atomic is hidden behind the loads of the current item instead of sitting between two items.
  if (tid == 0) s_misc[6] = first_item_id;
  for (int round = 0;; ++round) {
    __syncthreads();  // previous item's use of the ring / merge area is over; next id is visible
    const int item = s_misc[6 + (round & 1)];
    if (item >= total_items) break;

    // ---- decode the item ------------------------------------------------------------
    const int run = item / lanes_per_run;
    const int rem = item - run * lanes_per_run;
    const int hk = rem / p.n_hb;
    const int hbi = rem - hk * p.n_hb;
    int lo = 0, hi = p.batch - 1;  // largest b with s_prefix[b] <= run
    while (lo < hi) {
      int mid = (lo + hi + 1) >> 1;
      if (s_prefix[mid] <= run) lo = mid; else hi = mid - 1;
    }
    const int b = lo;
    const int len = max(s_lens[b], 0);
    const int tiles_b = (len + kTile - 1) / kTile;
    const int n_runs = s_prefix[b + 1] - s_prefix[b];
    const int j = run - s_prefix[b];
    const int run_tiles = (tiles_b + n_runs - 1) / n_runs;
    const int tile0 = min(j * run_tiles, tiles_b);
    const int tile1 = min(tile0 + run_tiles, tiles_b);
    const int n_tiles = tile1 - tile0;
    const int head0 = hk * p.group + hbi * p.hb;           // first q head of this item
    const int n_heads = min(p.hb, p.group - hbi * p.hb);   // q heads of this item

    // ---- q fragments (B operand of S^T = K Q^T) ---------------------------------------
    uint32_t qf[NT][kKSteps][2];
    float q_unscale[NT][2] = {};   // F8M: 1 / (scale q was multiplied by), for heads 2*t4, 2*t4+1
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const int hn = nt * 8 + g8;
      const bool ok = hn < n_heads;
      const size_t qoff = (size_t(b) * p.heads + head0 + (ok ? hn : 0)) * D;
      if constexpr (F8M) {
        // B fragment of m16n8k32: b0 = dims 32j+4t..+3, b1 = dims 32j+16+4t..+3 of head g8.
        // qf[nt][2j][0/1] = hi bytes of (b0, b1), qf[nt][2j+1][0/1] = lo bytes.
        float f[D / 32][8];
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < D / 32; ++j)
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const int d = j * 32 + (e >> 2) * 16 + t4 * 4 + (e & 3);
            float x = 0.f;
            if (ok) x = p.q_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.q)[qoff + d])
                                    : __half2float(reinterpret_cast<const __half*>(p.q)[qoff + d]);
            f[j][e] = x;
            amax = fmaxf(amax, fabsf(x));
          }
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const float sq = 384.f / fmaxf(amax, 1e-20f);      // head g8: |q * sq| <= 384 < 448
        const float inv = 1.f / sq;
        q_unscale[nt][0] = __shfl_sync(0xffffffffu, inv, (2 * t4) * 4);
        q_unscale[nt][1] = __shfl_sync(0xffffffffu, inv, (2 * t4 + 1) * 4);
#pragma unroll
        for (int j = 0; j < D / 32; ++j) {
          uint32_t h[4], l[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) split_e4m3x2(f[j][2 * e] * sq, f[j][2 * e + 1] * sq, h[e], l[e]);
          qf[nt][2 * j][0] = h[0] | (h[1] << 16);
          qf[nt][2 * j][1] = h[2] | (h[3] << 16);
          qf[nt][2 * j + 1][0] = l[0] | (l[1] << 16);
          qf[nt][2 * j + 1][1] = l[2] | (l[3] << 16);
        }
      } else
#pragma unroll
      for (int ks = 0; ks < kKSteps; ++ks) {
        if constexpr (!FP8) {
          const T* qp = reinterpret_cast<const T*>(p.q) + qoff + ks * 16 + t4 * 2;
          qf[nt][ks][0] = ok ? *reinterpret_cast<const uint32_t*>(qp) : 0u;
          qf[nt][ks][1] = ok ? *reinterpret_cast<const uint32_t*>(qp + 8) : 0u;
        } else {
          // k index 2t,2t+1 <-> d = 16ks+4t+{0,1}; k index 2t+8,2t+9 <-> d = 16ks+4t+{2,3}
          float f[4] = {0.f, 0.f, 0.f, 0.f};
          if (ok) {
            if (p.q_is_bf16) {
              const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + qoff + ks * 16 + t4 * 4;
#pragma unroll
              for (int e = 0; e < 4; ++e) f[e] = __bfloat162float(qp[e]);
            } else {
              const __half* qp = reinterpret_cast<const __half*>(p.q) + qoff + ks * 16 + t4 * 4;
#pragma unroll
              for (int e = 0; e < 4; ++e) f[e] = __half2float(qp[e]);
            }
          }
          qf[nt][ks][0] = pack2<__half>(f[0], f[1]);
          qf[nt][ks][1] = pack2<__half>(f[2], f[3]);
        }
      }
    }

    // ---- tile loader -----------------------------------------------------------------
    const unsigned char* kbase = reinterpret_cast<const unsigned char*>(p.k) +
                                 (size_t(hk) * p.head_stride + (p.bt ? 0 : size_t(b) * p.batch_stride)) * C::kEsize;
    const unsigned char* vbase = reinterpret_cast<const unsigned char*>(p.v) +
                                 (size_t(hk) * p.head_stride + (p.bt ? 0 : size_t(b) * p.batch_stride)) * C::kEsize;
    const int32_t* bt_row = p.bt ? p.bt + size_t(b) * p.bt_stride : nullptr;
    const size_t tok_bytes = size_t(p.tok_stride) * C::kEsize;
    const int ld_chunk = tid % C::kChunksPerRow;
    const int ld_row0 = tid / C::kChunksPerRow;
    constexpr int kRowsPerPass = kThreads / C::kChunksPerRow;
    constexpr int kPasses = kTile / kRowsPerPass;

    // block-table entry of the next tile to be issued, fetched one tile ahead (fast path)
    int32_t next_entry = 0;
    auto fetch_entry = [&](int tile) {
      if (bt_row && p.tile_in_page && tile < tile1) next_entry = bt_row[(tile * kTile) / p.page_size];
    };
    fetch_entry(tile0);

    auto issue_tile = [&](int tile, int stage) {
      const int tok0 = tile * kTile;
      const uint32_t sk = ring_u32 + stage * C::kStageBytes;
      const uint32_t sv = sk + C::kTileBytes;
      int64_t phys0 = tok0;  // contiguous cache: physical == logical
      int32_t page_entry = 0;
      if (bt_row && p.tile_in_page) {
        page_entry = next_entry;
        phys0 = int64_t(page_entry) * p.page_size + (tok0 % p.page_size);
        fetch_entry(tile + 1);
      }
#pragma unroll
      for (int i = 0; i < kPasses; ++i) {
        const int row = ld_row0 + i * kRowsPerPass;
        const int tok = tok0 + row;
        const bool ok = tok < len;
        int64_t phys = phys0 + row;
        if (bt_row && !p.tile_in_page) {
          phys = ok ? int64_t(bt_row[tok / p.page_size]) * p.page_size + (tok % p.page_size) : 0;
        }
        const size_t off = ok ? size_t(phys) * tok_bytes + ld_chunk * 16 : 0;
        const uint32_t d = row * C::kRowStride + ld_chunk * 16;
        cp_async_16(sk + d, kbase + off, ok ? 16 : 0);
        cp_async_16(sv + d, vbase + off, ok ? 16 : 0);
      }
      if constexpr (FP8) {
        if (tid < kTile) {
          const int tok = tok0 + tid;
          const bool ok = tok < len;
          int32_t pg = page_entry;
          if (!p.tile_in_page || !bt_row) {
            pg = ok ? (bt_row ? bt_row[tok / p.page_size]
                              : int32_t((size_t(b) * (p.batch_stride / p.tok_stride) + tok) / p.page_size))
                    : 0;
          }
          const size_t so = ok ? size_t(pg) * p.heads_kv + hk : 0;
          const uint32_t ss = sk + 2 * C::kTileBytes + tid * 4;
          cp_async_4(ss, p.k_scale + so, ok ? 4 : 0);
          cp_async_4(ss + kTile * 4, p.v_scale + so, ok ? 4 : 0);
        }
      }
    };

#if TB200_DEC_PREFETCH_NEXT
    // (sequence, KV head, first tile, end tile, length) of the CTA's next item, or false.  The id was
    // requested before this item's tile loop; it is visible after the loop's first barrier.
    auto next_item_desc = [&](int& nb, int& nhk, int& nt0, int& nt1, int& nlen) -> bool {
      const int nitem = s_misc[6 + ((round + 1) & 1)];
      if (nitem >= total_items) return false;
      const int nrun = nitem / lanes_per_run;
      nhk = (nitem - nrun * lanes_per_run) / p.n_hb;
      int lo2 = 0, hi2 = p.batch - 1;
      while (lo2 < hi2) {
        const int mid = (lo2 + hi2 + 1) >> 1;
        if (s_prefix[mid] <= nrun) lo2 = mid; else hi2 = mid - 1;
      }
      nb = lo2;
      nlen = max(s_lens[nb], 0);
      const int ntiles = (nlen + kTile - 1) / kTile;
      const int nruns = s_prefix[nb + 1] - s_prefix[nb];
      const int nrt = (ntiles + nruns - 1) / nruns;
      nt0 = min((nrun - s_prefix[nb]) * nrt, ntiles);
      nt1 = min(nt0 + nrt, ntiles);
      return nt1 > nt0;
    };
    // Only where a tile lies inside one page (or there is no table), and only for items long enough
    // that the table entries fetched at the first iteration have landed by the time they are used.
    const bool prefetch_ok = (!bt_row || p.tile_in_page) && n_tiles >= 2 * (C::kStages - 1);
    const int prefetch_at = n_tiles - (C::kStages - 1);      // first iteration with no load left to issue
#endif

    // ---- running state ----------------------------------------------------------------
    float oacc[NT][kKSteps][4];
    float m_run[NT][2], l_run[NT][2];
    float v_unit = 1.f;   // F8M: V scale that oacc is currently expressed in
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      m_run[nt][0] = m_run[nt][1] = kNegFloor;
      l_run[nt][0] = l_run[nt][1] = 0.f;
#pragma unroll
      for (int mt = 0; mt < kKSteps; ++mt)
#pragma unroll
        for (int e = 0; e < 4; ++e) oacc[nt][mt][e] = 0.f;
    }

#pragma unroll
    for (int s = 0; s < C::kStages - 1; ++s) {
      if (s < n_tiles) issue_tile(tile0 + s, s);
      cp_async_commit();
    }
    if (tid == 0) s_misc[6 + ((round + 1) & 1)] = atomicAdd(&p.counters[0], 1);  // id of the next item
#if TB200_DEC_DEFER
    resolve_pending();  // ticket / merge of the previous item, under this item's first loads
#endif

    for (int it = 0; it < n_tiles; ++it) {
      cp_async_wait<C::kStages - 2>();
      __syncthreads();
      {
        const int nx = it + C::kStages - 1;
        if (nx < n_tiles) issue_tile(tile0 + nx, nx % C::kStages);
#if TB200_DEC_PREFETCH_NEXT
        if (prefetch_ok && it == 0 && p.bt && tid < C::kStages - 1) {
          // block-table entries of the next item's first tiles: asynchronous 4-byte copies that ride
          // in this iteration's group, so no thread waits for them
          int nb, nhk, nt0, nt1, nlen;
          if (next_item_desc(nb, nhk, nt0, nt1, nlen) && nt0 + tid < nt1)
            cp_async_4(smem_u32(&s_misc[8 + tid]),
                       p.bt + size_t(nb) * p.bt_stride + ((nt0 + tid) * kTile) / p.page_size, 4);
        }
#endif
        cp_async_commit();
      }
#if TB200_DEC_PREFETCH_NEXT
      if (prefetch_ok && it == prefetch_at) {
        int nb, nhk, nt0, nt1, nlen;
        if (next_item_desc(nb, nhk, nt0, nt1, nlen)) {
          constexpr int kLines = C::kRowBytes >= 128 ? C::kRowBytes / 128 : 1;   // 128-byte lines per token row
          const size_t head_off = (size_t(nhk) * p.head_stride + (p.bt ? 0 : size_t(nb) * p.batch_stride)) * C::kEsize;
          const unsigned char* nk = reinterpret_cast<const unsigned char*>(p.k) + head_off;
          const unsigned char* nv = reinterpret_cast<const unsigned char*>(p.v) + head_off;
#pragma unroll 1
          for (int st2 = 0; st2 < C::kStages - 1; ++st2) {
            const int tile = nt0 + st2;
            if (tile >= nt1) break;
            const int tok0 = tile * kTile;
            const int64_t phys0 = p.bt ? int64_t(s_misc[8 + st2]) * p.page_size + (tok0 % p.page_size) : tok0;
            for (int idx = tid; idx < kTile * kLines; idx += kThreads) {
              const int row = idx / kLines, line = idx % kLines;
              if (tok0 + row < nlen) {
                const size_t off = size_t(phys0 + row) * tok_bytes + line * 128;
                asm volatile("prefetch.global.L2 [%0];" ::"l"(nk + off));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(nv + off));
              }
            }
          }
        }
      }
#endif
      const int stage = it % C::kStages;
      const uint32_t st_base = ring_u32 + stage * C::kStageBytes;
      const int tok_a = (tile0 + it) * kTile + warp * 16 + g8;  // token of c0/c1; c2/c3 is +8

      // ---- S^T = K Q^T  (16 tokens x 8*NT heads per warp) ---------------------------
      // two accumulators per score tile (even / odd k-steps) halve the dependent MMA chain
      float sacc[NT][4], sacc2[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) { sacc[nt][e] = 0.f; sacc2[nt][e] = 0.f; }

      if constexpr (!FP8) {
#pragma unroll
        for (int ks = 0; ks < kKSteps; ++ks) {
          uint32_t a[4];
          ldmatrix_x4(a, st_base + k_lane_off + ks * 32);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_16816<T>((ks & 1) ? sacc2[nt] : sacc[nt], a, qf[nt][ks]);
        }
      } else if constexpr (F8M) {
#pragma unroll
        for (int jj = 0; jj < D / 32; ++jj) {
          // the four 8x16-byte blocks are exactly the A fragment of m16n8k32 (16 tokens x 32 dims)
          uint32_t r[4];
          ldmatrix_x4(r, st_base + k_lane_off + jj * 32);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_16832_e4m3(sacc[nt], r, qf[nt][2 * jj]);       // K q_hi^T
            mma_16832_e4m3(sacc2[nt], r, qf[nt][2 * jj + 1]);  // K q_lo^T
          }
        }
      } else {
#pragma unroll
        for (int jj = 0; jj < D / 32; ++jj) {
          uint32_t r[4];
          ldmatrix_x4(r, st_base + k_lane_off + jj * 32);
          uint32_t a0[4] = {e4m3x2_to_f16x2_scaled<0x1404>(r[0]), e4m3x2_to_f16x2_scaled<0x1404>(r[1]),
                            e4m3x2_to_f16x2_scaled<0x3424>(r[0]), e4m3x2_to_f16x2_scaled<0x3424>(r[1])};
          uint32_t a1[4] = {e4m3x2_to_f16x2_scaled<0x1404>(r[2]), e4m3x2_to_f16x2_scaled<0x1404>(r[3]),
                            e4m3x2_to_f16x2_scaled<0x3424>(r[2]), e4m3x2_to_f16x2_scaled<0x3424>(r[3])};
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_16816<T>(sacc[nt], a0, qf[nt][2 * jj]);
            mma_16816<T>(sacc2[nt], a1, qf[nt][2 * jj + 1]);
          }
        }
      }

      // ---- scale, softcap, mask, online softmax ----------------------------------------
      float sc_lo = qk_scale, sc_hi = qk_scale;  // per-token score scale (rows g8 and g8+8)
      float vs_lo = 1.f, vs_hi = 1.f;
      float unit_fix = 1.f;   // F8M: factor that moves O from the previous tile's V scale to this one's
      if constexpr (FP8) {
        const float* s_ks = reinterpret_cast<const float*>(ring + stage * C::kStageBytes + 2 * C::kTileBytes);
        const float* s_vs = s_ks + kTile;
        if constexpr (F8M) {
          sc_lo *= s_ks[warp * 16 + g8];
          sc_hi *= s_ks[warp * 16 + g8 + 8];
          // O is kept in units of the current tile's V scale (one scale per tile: the tile lies in
          // one page); a slice with no live token (scale loaded as 0) leaves the unit alone
          const float vs = s_vs[warp * 16];
          if (vs > 0.f) { unit_fix = v_unit / vs; v_unit = vs; }
          vs_lo = vs_hi = 256.f;    // P enters the MMA as p * 256 <= 256 (e4m3 holds up to 448)
        } else {
          sc_lo *= s_ks[warp * 16 + g8] * kE4m3Unit;
          sc_hi *= s_ks[warp * 16 + g8 + 8] * kE4m3Unit;
          vs_lo = s_vs[warp * 16 + g8] * kE4m3Unit;
          vs_hi = s_vs[warp * 16 + g8 + 8] * kE4m3Unit;
        }
      }
      const bool ok_lo = tok_a < len, ok_hi = tok_a + 8 < len;
      uint32_t pb[NT][2];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        float s0 = (sacc[nt][0] + sacc2[nt][0]) * sc_lo, s1 = (sacc[nt][1] + sacc2[nt][1]) * sc_lo;
        float s2 = (sacc[nt][2] + sacc2[nt][2]) * sc_hi, s3 = (sacc[nt][3] + sacc2[nt][3]) * sc_hi;
        if constexpr (F8M) {
          s0 *= q_unscale[nt][0]; s1 *= q_unscale[nt][1];
          s2 *= q_unscale[nt][0]; s3 *= q_unscale[nt][1];
        }
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
        const float mn0 = fmaxf(m_run[nt][0], mx0), mn1 = fmaxf(m_run[nt][1], mx1);
        const float al0 = fast_exp2(m_run[nt][0] - mn0), al1 = fast_exp2(m_run[nt][1] - mn1);
        const float oa0 = F8M ? al0 * unit_fix : al0, oa1 = F8M ? al1 * unit_fix : al1;
        m_run[nt][0] = mn0; m_run[nt][1] = mn1;
        const float p0 = fast_exp2(s0 - mn0), p1 = fast_exp2(s1 - mn1);
        const float p2 = fast_exp2(s2 - mn0), p3 = fast_exp2(s3 - mn1);
        l_run[nt][0] = l_run[nt][0] * al0 + p0 + p2;
        l_run[nt][1] = l_run[nt][1] * al1 + p1 + p3;
#pragma unroll
        for (int mt = 0; mt < kKSteps; ++mt) {
          oacc[nt][mt][0] *= oa0; oacc[nt][mt][1] *= oa1;
          oacc[nt][mt][2] *= oa0; oacc[nt][mt][3] *= oa1;
        }
        if constexpr (F8M) {
          // B fragment of m16n8k32: b0 = P_hi, b1 = P_lo of head g8 for the four tokens
          // (2t, 2t+1, 8+2t, 9+2t), the order in which the V fragment below lists its tokens.
          // x: byte pairs (head 2t, 2t+1) of token g8 (low half) and token g8+8 (high half);
          // after the 8x8 transpose an even-g8 lane holds tokens 2t, 2t+1 and its odd neighbour
          // tokens 8+2t, 9+2t, both for the head pair g8>>1; one exchange completes each lane.
          uint32_t h01, l01, h23, l23;
          split_e4m3x2(p0 * vs_lo, p1 * vs_lo, h01, l01);
          split_e4m3x2(p2 * vs_hi, p3 * vs_hi, h23, l23);
          const uint32_t xh = movmatrix_trans(h01 | (h23 << 16));
          const uint32_t xl = movmatrix_trans(l01 | (l23 << 16));
          const uint32_t yh = __shfl_xor_sync(0xffffffffu, xh, 4);
          const uint32_t yl = __shfl_xor_sync(0xffffffffu, xl, 4);
          const bool odd = g8 & 1;
          pb[nt][0] = odd ? prmt(yh, xh, 0x7531) : prmt(xh, yh, 0x6420);
          pb[nt][1] = odd ? prmt(yl, xl, 0x7531) : prmt(xl, yl, 0x6420);
        } else {
          // P^T as the B operand: transpose the two 8x8 (token x head) blocks across the warp
          pb[nt][0] = movmatrix_trans(pack2<T>(p0 * vs_lo, p1 * vs_lo));
          pb[nt][1] = movmatrix_trans(pack2<T>(p2 * vs_hi, p3 * vs_hi));
        }
      }

      // ---- O^T += V^T P^T ------------------------------------------------------------------
      if constexpr (!FP8) {
#pragma unroll
        for (int mt = 0; mt < kKSteps; ++mt) {
          uint32_t a[4];
          ldmatrix_x4_trans(a, st_base + v_lane_off + mt * 32);
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) mma_16816<T>(oacc[nt][mt], a, pb[nt]);
        }
      } else if constexpr (F8M) {
#pragma unroll
        for (int ii = 0; ii < D / 32; ++ii) {
          // r[0], r[1]: tokens 0-7, 8-15 at dims 32ii..+15; r[2], r[3]: the same tokens, next 16 dims.
          // Each register is 2 tokens x 2 dims: bytes (0,2) dim 2*g8, bytes (1,3) dim 2*g8+1.
          uint32_t r[4];
          ldmatrix_x4_trans(r, st_base + v_lane_off + ii * 32);
          uint32_t a0[4], a1[4];
          a0[0] = prmt(r[0], r[1], 0x6420); a0[1] = prmt(r[0], r[1], 0x7531);
          a1[0] = prmt(r[2], r[3], 0x6420); a1[1] = prmt(r[2], r[3], 0x7531);
          a0[2] = a0[0]; a0[3] = a0[1];     // k slots 16..31 repeat the 16 tokens: they meet P_lo
          a1[2] = a1[0]; a1[3] = a1[1];
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_16832_e4m3(oacc[nt][2 * ii], a0, pb[nt]);
            mma_16832_e4m3(oacc[nt][2 * ii + 1], a1, pb[nt]);
          }
        }
      } else {
#pragma unroll
        for (int ii = 0; ii < D / 32; ++ii) {
          uint32_t r[4];
          ldmatrix_x4_trans(r, st_base + v_lane_off + ii * 32);
          // register = 2 tokens x 2 dims; bytes (0,2) are dim 2*g8, bytes (1,3) dim 2*g8+1
          uint32_t a0[4] = {e4m3x2_to_f16x2_scaled<0x2404>(r[0]), e4m3x2_to_f16x2_scaled<0x3414>(r[0]),
                            e4m3x2_to_f16x2_scaled<0x2404>(r[1]), e4m3x2_to_f16x2_scaled<0x3414>(r[1])};
          uint32_t a1[4] = {e4m3x2_to_f16x2_scaled<0x2404>(r[2]), e4m3x2_to_f16x2_scaled<0x3414>(r[2]),
                            e4m3x2_to_f16x2_scaled<0x2404>(r[3]), e4m3x2_to_f16x2_scaled<0x3414>(r[3])};
#pragma unroll
          for (int nt = 0; nt < NT; ++nt) {
            mma_16816<T>(oacc[nt][2 * ii], a0, pb[nt]);
            mma_16816<T>(oacc[nt][2 * ii + 1], a1, pb[nt]);
          }
        }
      }
    }
    cp_async_wait<0>();
    __syncthreads();  // ring is free: reuse it as the cross-warp merge area

    // ---- the 4 warps meet: per-warp (m, l, O^T) -> shared memory ---------------------------
    float* s_o = reinterpret_cast<float*>(smem);                          // [warp][8*NT][kOStride]
    float* s_ml = s_o + kWarps * (8 * NT) * C::kOStride;                  // [warp][8*NT][2]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      float l0 = l_run[nt][0], l1 = l_run[nt][1];
#pragma unroll
      for (int o = 4; o < 32; o <<= 1) {
        l0 += __shfl_xor_sync(0xffffffffu, l0, o);
        l1 += __shfl_xor_sync(0xffffffffu, l1, o);
      }
      const int h0 = nt * 8 + t4 * 2;
      if (g8 == 0) {
        float* ml = s_ml + (warp * (8 * NT) + h0) * 2;
        ml[0] = m_run[nt][0]; ml[1] = l0; ml[2] = m_run[nt][1]; ml[3] = l1;
      }
      float* so0 = s_o + (warp * (8 * NT) + h0) * C::kOStride;
      float* so1 = so0 + C::kOStride;
#pragma unroll
      for (int mt = 0; mt < kKSteps; ++mt) {
        // fragment rows -> head dims: 16-bit path rows g8, g8+8 of the m-tile; FP8 path the
        // ldmatrix on byte pairs interleaves them: rows g8, g8+8 are dims 2*g8, 2*g8+1
        const int d_lo = FP8 ? mt * 16 + 2 * g8 : mt * 16 + g8;
        const int d_hi = FP8 ? d_lo + 1 : d_lo + 8;
        const float of = F8M ? v_unit * (1.f / 256.f) : 1.f;
        so0[d_lo] = oacc[nt][mt][0] * of; so1[d_lo] = oacc[nt][mt][1] * of;
        so0[d_hi] = oacc[nt][mt][2] * of; so1[d_hi] = oacc[nt][mt][3] * of;
      }
    }
    __syncthreads();

    const bool single = (n_runs == 1);
    float* po = p.part_o + size_t(item) * p.hb * D;
    float* pml = p.part_ml + size_t(item) * p.hb * 2;
    for (int idx = tid; idx < n_heads * D; idx += kThreads) {
      const int hn = idx / D, d = idx - hn * D;
      float mw[kWarps], M = kNegFloor;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        mw[w] = s_ml[(w * (8 * NT) + hn) * 2];
        M = fmaxf(M, mw[w]);
      }
      float acc = 0.f, L = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float e = fast_exp2(mw[w] - M);
        acc += e * s_o[(w * (8 * NT) + hn) * C::kOStride + d];
        L += e * s_ml[(w * (8 * NT) + hn) * 2 + 1];
      }
      if (single) {
        const size_t orow = size_t(b) * p.heads + head0 + hn;
        emit_out<TO>(p, parity, orow, d, D, L > 0.f ? acc / L : 0.f);
        if (d == 0) emit_lse(p, parity, orow, D, L > 0.f ? M + log2f(L) : -INFINITY);
      } else {
        po[hn * D + d] = acc;
        if (d == 0) { pml[hn * 2] = M; pml[hn * 2 + 1] = L; }
      }
    }
    if (!single) {
      // the ticket for this (sequence, KV head, head block) is taken at the start of the next
      // item, after that item's first loads are in flight
      pend.valid = true;
      pend.ticket = p.counters + kCounterWords + (size_t(b) * p.heads_kv + hk) * p.n_hb + hbi;
      pend.n_runs = n_runs;
      pend.first_item = s_prefix[b] * lanes_per_run + rem;
      pend.b = b; pend.head0 = head0; pend.n_heads = n_heads;
    }
#if !TB200_DEC_DEFER
    __syncthreads();
    resolve_pending();
#endif
  }
  resolve_pending();

  // ---- the last CTA to leave resets the scheduler counters ------------------------------
  if (p.world > 1) {
    // every thread pushes its stores to the other GPUs out to system scope before the CTA reports
    __threadfence_system();
    __syncthreads();
  }
  if (tid == 0) {
    __threadfence();
    const int done = atomicAdd(&p.counters[1], 1);
    if (done == int(gridDim.x) - 1) {
      p.counters[0] = 0;
      p.counters[1] = 0;
      __threadfence();
      if (p.world > 1) {
        // all CTAs of this launch have reported: every rank's copy of this rank's result is complete
        *p.step_counter = step;
        // ONE system-scope fence, then relaxed flag stores: a release store per peer would be a fence per peer
        // (eight in a row at eight ranks, on the critical path of the step)
        __threadfence_system();
        for (int r = 0; r < p.world; ++r)
          asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p.peer_flag[r]), "r"(step) : "memory");
      }
    }
  }
}

// ---- host side ------------------------------------------------------------------------------

template <int D, bool FP8, typename T, int NT, typename TO, bool F8M = false, bool WIDE = false>
int launch(const DecodeParams& p, cudaStream_t stream) {
  auto kern = gqa_decode_kernel<D, FP8, T, NT, TO, F8M, WIDE>;
  const size_t smem = smem_bytes<D, FP8, WIDE>(p.batch, NT);
  // per device: the largest dynamic shared memory size configured so far, and the number of CTAs an
  // SM holds at the size of the last launch (the grid is one CTA per resident slot: a CTA that starts
  // late finds the item queue empty and only costs its plan)
  static thread_local size_t configured[64] = {0};
  static thread_local size_t sized_for[64] = {0};
  static thread_local int resident[64] = {0};
  int dev = 0;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) TB200_FAIL(TB200_ERR_UNSUPPORTED, "device index %d is outside [0, 64)", dev);
  if (configured[dev] < smem) {
    TB200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  if (sized_for[dev] != smem) {
    int n = 0;
    TB200_CUDA_CHECK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kThreads, smem));
    if (n <= 0) TB200_FAIL(TB200_ERR_UNSUPPORTED, "the decode kernel does not fit an SM with %zu bytes of shared memory", smem);
    sized_for[dev] = smem;
    resident[dev] = n < min_blocks(FP8, NT, WIDE) ? n : min_blocks(FP8, NT, WIDE);
  }
  kern<<<sm_count() * resident[dev], kThreads, smem, stream>>>(p);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}

template <int D, bool FP8, typename T, int NT, bool F8M = false, bool WIDE = false>
int launch_o(const DecodeParams& p, int o_dtype, cudaStream_t s) {
  switch (o_dtype) {
    case TB200_F32: return launch<D, FP8, T, NT, float, F8M, WIDE>(p, s);
    case TB200_BF16: return launch<D, FP8, T, NT, __nv_bfloat16, F8M, WIDE>(p, s);
    case TB200_F16: return launch<D, FP8, T, NT, __half, F8M, WIDE>(p, s);
  }
  TB200_FAIL(TB200_ERR_UNSUPPORTED, "o_dtype %d is not F16, BF16 or F32", o_dtype);
}

template <int D, int NT>
int launch_t(const DecodeParams& p, int q_dtype, int kv_dtype, int o_dtype, bool wide, bool fp8_mma, cudaStream_t s) {
  if (kv_dtype == TB200_E4M3) {
    // The f16 expansion path is the default: on B200 the e4m3 mma.sync path measured slower
    // (3.7 vs 4.4 TB/s on 128 x 4096-token sequences).  TB200_DECODE_FP8_MMA selects it where
    // its precondition holds (one scale per tile, i.e. page_size a multiple of 64).
    if (p.tile_in_page && fp8_mma) return launch_o<D, true, __half, NT, true>(p, o_dtype, s);
    return launch_o<D, true, __half, NT>(p, o_dtype, s);
  }
  if constexpr (NT == 1) {
    if (wide) {
      if (q_dtype == TB200_BF16) return launch_o<D, false, __nv_bfloat16, NT, false, true>(p, o_dtype, s);
      return launch_o<D, false, __half, NT, false, true>(p, o_dtype, s);
    }
  }
  if (q_dtype == TB200_BF16) return launch_o<D, false, __nv_bfloat16, NT>(p, o_dtype, s);
  return launch_o<D, false, __half, NT>(p, o_dtype, s);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_gqa_decode_workspace_bytes(int batch, int heads, int heads_kv, int dim) {
  if (batch <= 0 || heads <= 0 || heads_kv <= 0 || dim <= 0 || heads % heads_kv != 0) return 0;
  return make_layout(batch, heads, heads_kv, dim).total;
}

namespace {
// which kernel served this thread's last decode call (tb200_gqa_decode_last_kernel)
thread_local int t_last_kernel = 0;
struct PeerTargets {
  int world, rank;
  void* const* buffers;   // [world] base of every rank's exchange buffer, as mapped into this process
  int* const* flags;      // [world] this rank's flag word on every rank
  int* step_counter;      // local device int
};

int decode_impl(const void* q, const void* k, const void* v, void* o, float* lse,
                const int32_t* real_seqlen_kv, int32_t uniform_seqlen,
                const int32_t* block_table, int32_t block_table_stride,
                const float* k_scale, const float* v_scale,
                int q_dtype, int kv_dtype, int o_dtype,
                int batch, int heads, int heads_kv, int dim, int page_size,
                int64_t kv_token_stride, int64_t kv_head_stride, int64_t kv_batch_stride,
                float sm_scale, float softcap, int64_t kv_pool_tokens, int flags,
                void* workspace, size_t workspace_bytes, void* stream, const PeerTargets* peers) {
  if (!q || !k || !v || (!o && !peers)) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "q, k, v and o must be non-null");
  if (batch <= 0 || heads <= 0 || heads_kv <= 0 || dim <= 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "batch, heads, heads_kv and dim must be positive");
  if (heads % heads_kv != 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "heads must be divisible by heads_kv");
  if (batch > kMaxBatch) TB200_FAIL(TB200_ERR_UNSUPPORTED, "batch %d exceeds %d", batch, kMaxBatch);
  if (q_dtype != TB200_F16 && q_dtype != TB200_BF16)
    TB200_FAIL(TB200_ERR_UNSUPPORTED, "q_dtype must be F16 or BF16");
  if (kv_dtype != q_dtype && kv_dtype != TB200_E4M3)
    TB200_FAIL(TB200_ERR_UNSUPPORTED, "kv_dtype must equal q_dtype or be E4M3");
  if (o_dtype != q_dtype && o_dtype != TB200_F32)
    TB200_FAIL(TB200_ERR_UNSUPPORTED, "o_dtype must equal q_dtype or be F32");
  if (kv_dtype == TB200_E4M3 && (!k_scale || !v_scale))
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "an E4M3 cache needs k_scale and v_scale");
  if (block_table || kv_dtype == TB200_E4M3) {
    if (page_size <= 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "page_size must be positive");
  }
  if (block_table && block_table_stride <= 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "block_table_stride must be positive");
  if (!real_seqlen_kv && uniform_seqlen < 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "uniform_seqlen must be non-negative");
  if (softcap < 0.f) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "softcap must be non-negative");
  if (dim != 64 && dim != 128) TB200_FAIL(TB200_ERR_UNSUPPORTED, "head dim %d (supported: 64, 128)", dim);
  const int esize = kv_dtype == TB200_E4M3 ? 1 : 2;
  if ((kv_token_stride * esize) % 16 != 0 || (kv_head_stride * esize) % 16 != 0 ||
      (kv_batch_stride * esize) % 16 != 0 || (reinterpret_cast<uintptr_t>(k) & 15) ||
      (reinterpret_cast<uintptr_t>(v) & 15) || (reinterpret_cast<uintptr_t>(q) & 7))
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "k/v base and strides must be 16-byte aligned (q 8-byte)");
  if (!block_table && kv_token_stride <= 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "kv_token_stride must be positive");
  if (flags < 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "flags must be a combination of TB200_DECODE_* values");

  const bool fp8 = kv_dtype == TB200_E4M3;
  const DecodeVariant var = parse_variant(flags);
  // tokens a sequence may hold, as far as the host can tell without reading the lengths
  const long long capacity = block_table ? (long long)block_table_stride * (page_size > 0 ? page_size : 1)
                             : real_seqlen_kv ? (kv_token_stride > 0 ? kv_batch_stride / kv_token_stride : 0)
                                              : (long long)uniform_seqlen;
  bool wide = !fp8 && heads / heads_kv <= 8 && capacity >= 16384;
  if (var.wide >= 0) wide = !fp8 && heads / heads_kv <= 8 && var.wide == 1;
  const Layout L = make_layout(batch, heads, heads_kv, dim);
  if (!workspace || workspace_bytes < L.total || (reinterpret_cast<uintptr_t>(workspace) & 255))
    TB200_FAIL(TB200_ERR_WORKSPACE, "workspace must be 256-byte aligned and hold %zu bytes (got %zu)",
               L.total, workspace_bytes);

  DecodeParams p{};
  p.q = q; p.k = k; p.v = v; p.o = o; p.lse = lse;
  p.lens = real_seqlen_kv; p.uniform_len = uniform_seqlen;
  p.bt = block_table; p.bt_stride = block_table_stride;
  p.k_scale = k_scale; p.v_scale = v_scale;
  p.batch = batch; p.heads = heads; p.heads_kv = heads_kv; p.group = heads / heads_kv;
  p.hb = L.hb; p.n_hb = L.n_hb;
  p.page_size = page_size > 0 ? page_size : 1;
  p.tile_in_page = (block_table && page_size % kTile == 0) ? 1 : 0;
  p.tok_stride = kv_token_stride; p.head_stride = kv_head_stride; p.batch_stride = kv_batch_stride;
  p.sm_scale = sm_scale; p.softcap = softcap;
  p.q_is_bf16 = q_dtype == TB200_BF16;
  p.target_items = L.target_items; p.max_items = L.max_items;
  p.force_chunk = var.chunk_tiles;
  p.wait_cycles = 1000000000LL;   // ~0.5 s
  if (peers) {
    p.world = peers->world; p.rank = peers->rank; p.step_counter = peers->step_counter;
    p.slot_floats = (long long)batch * heads * (dim + 1);
    for (int r = 0; r < peers->world; ++r) {
      p.peer_o[r] = static_cast<float*>(peers->buffers[r]);
      p.peer_flag[r] = peers->flags[r];
    }
  }
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  p.counters = reinterpret_cast<int*>(ws);
  p.part_o = reinterpret_cast<float*>(ws + L.counters_bytes);
  p.part_ml = reinterpret_cast<float*>(ws + L.counters_bytes + L.part_o_bytes);

  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The TMA kernel serves caches whose 64-token tiles are contiguous or whole pages (no table, pages that
  // are multiples of 64 tokens, pages of 16 or 32) with 128- or 256-byte token rows and up to 8 q heads per KV head; it
  // declines everything else, and the cp.async kernel below serves every layout.
  if (!var.no_tma && !var.fp8_mma && var.wide != 1) {
    const int st = launch_decode_tma(p, q_dtype, kv_dtype, o_dtype, dim, L.nt, kv_pool_tokens, s);
    if (st != kTmaNotApplicable) {
      if (st == TB200_OK) t_last_kernel = TB200_DECODE_KERNEL_TMA;
      return st;
    }
  }
  t_last_kernel = TB200_DECODE_KERNEL_CP_ASYNC;
  if (dim == 128)
    return L.nt == 1 ? launch_t<128, 1>(p, q_dtype, kv_dtype, o_dtype, wide, var.fp8_mma, s)
                     : launch_t<128, 2>(p, q_dtype, kv_dtype, o_dtype, wide, var.fp8_mma, s);
  return L.nt == 1 ? launch_t<64, 1>(p, q_dtype, kv_dtype, o_dtype, wide, var.fp8_mma, s)
                   : launch_t<64, 2>(p, q_dtype, kv_dtype, o_dtype, wide, var.fp8_mma, s);
}
}  // namespace

extern "C" int tb200_gqa_decode_last_kernel(void) { return t_last_kernel; }

extern "C" int tb200_gqa_decode(const void* q, const void* k, const void* v, void* o, float* lse,
                                const int32_t* real_seqlen_kv, int32_t uniform_seqlen,
                                const int32_t* block_table, int32_t block_table_stride,
                                const float* k_scale, const float* v_scale,
                                int q_dtype, int kv_dtype, int o_dtype,
                                int batch, int heads, int heads_kv, int dim, int page_size,
                                int64_t kv_token_stride, int64_t kv_head_stride, int64_t kv_batch_stride,
                                float sm_scale, float softcap, int64_t kv_pool_tokens, int flags,
                                void* workspace, size_t workspace_bytes, void* stream) {
  return decode_impl(q, k, v, o, lse, real_seqlen_kv, uniform_seqlen, block_table, block_table_stride, k_scale,
                     v_scale, q_dtype, kv_dtype, o_dtype, batch, heads, heads_kv, dim, page_size, kv_token_stride,
                     kv_head_stride, kv_batch_stride, sm_scale, softcap, kv_pool_tokens, flags, workspace,
                     workspace_bytes, stream, nullptr);
}

extern "C" int tb200_gqa_decode_sharded(const void* q, const void* k, const void* v,
                                        const int32_t* real_seqlen_kv, int32_t uniform_seqlen,
                                        const int32_t* block_table, int32_t block_table_stride,
                                        const float* k_scale, const float* v_scale, int q_dtype, int kv_dtype,
                                        int batch, int heads, int heads_kv, int dim, int page_size,
                                        int64_t kv_token_stride, int64_t kv_head_stride, int64_t kv_batch_stride,
                                        float sm_scale, float softcap, int64_t kv_pool_tokens, int flags,
                                        void* const* peer_buffers,
                                        int* const* peer_flags, int* step_counter, int world, int rank,
                                        void* workspace, size_t workspace_bytes, void* stream) {
  if (world < 2 || world > kMaxPeers || rank < 0 || rank >= world)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "world must be 2..%d and rank inside it", kMaxPeers);
  if (!peer_buffers || !peer_flags || !step_counter)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "peer_buffers, peer_flags and step_counter must be non-null");
  for (int r = 0; r < world; ++r)
    if (!peer_buffers[r] || !peer_flags[r] || (reinterpret_cast<uintptr_t>(peer_buffers[r]) & 15))
      TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "peer buffer / flag %d is null or misaligned", r);
  const PeerTargets peers{world, rank, peer_buffers, peer_flags, step_counter};
  return decode_impl(q, k, v, nullptr, nullptr, real_seqlen_kv, uniform_seqlen, block_table, block_table_stride,
                     k_scale, v_scale, q_dtype, kv_dtype, TB200_F32, batch, heads, heads_kv, dim, page_size,
                     kv_token_stride, kv_head_stride, kv_batch_stride, sm_scale, softcap, kv_pool_tokens, flags,
                     workspace, workspace_bytes, stream, &peers);
}


// ---- decode for callers that cannot allocate device memory ---------------------------------------
//
// Some hosts of this library are not allowed to call cudaMalloc at the point where they decode: a
// serving runtime that hands every byte of the device to its own pool allocator at start-up and
// forbids driver allocations afterwards, or a plugin running inside somebody else's framework whose
// allocator it must not bypass.  For them the split-KV scratch (scheduler counters, merge tickets and
// fp32 partials) lives in a fixed array inside the library image instead of a caller-provided
// workspace.  The array costs kDecodeStaticScratchBytes of device memory on every GPU that loads the
// library, for the life of the process, whether this entry point is used or not.
constexpr size_t kDecodeStaticScratchBytes = size_t(24) << 20;
static __device__ __align__(256) unsigned char g_decode_static_scratch[kDecodeStaticScratchBytes];

namespace {
// Device address of g_decode_static_scratch on each device.  In host code the array's name is only
// a handle for the runtime, not an address a kernel can use; the real address differs per device
// and is looked up once, with that device current.
void* g_scratch_addr[64] = {nullptr};
}  // namespace

extern "C" int tb200_gqa_decode_noalloc(const void* q, const void* k, const void* v, void* o, float* lse,
                                        const int32_t* real_seqlen_kv, int32_t uniform_seqlen,
                                        const int32_t* block_table, int32_t block_table_stride,
                                        const float* k_scale, const float* v_scale,
                                        int q_dtype, int kv_dtype, int o_dtype,
                                        int batch, int heads, int heads_kv, int dim, int page_size,
                                        int64_t kv_token_stride, int64_t kv_head_stride, int64_t kv_batch_stride,
                                        float sm_scale, float softcap, void* stream) {
  if (batch <= 0 || heads <= 0 || heads_kv <= 0 || dim <= 0 || heads % heads_kv != 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "batch, heads, heads_kv and dim must be positive and heads divisible by heads_kv");
  // (the scratch layout is the same for every kernel variant the library may pick)
  const Layout L = make_layout(batch, heads, heads_kv, dim);
  if (L.total > kDecodeStaticScratchBytes)
    TB200_FAIL(TB200_ERR_WORKSPACE,
               "this problem needs %zu bytes of scratch but the built-in scratch holds %zu; use "
               "tb200_gqa_decode with a caller-provided workspace", L.total, kDecodeStaticScratchBytes);
  int dev = 0;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) TB200_FAIL(TB200_ERR_UNSUPPORTED, "device index %d is outside [0, 64)", dev);
  if (g_scratch_addr[dev] == nullptr) {
    void* addr = nullptr;
    TB200_CUDA_CHECK(cudaGetSymbolAddress(&addr, g_decode_static_scratch));
    g_scratch_addr[dev] = addr;
  }
  // The array keeps whatever the previous call left: partials of another shape may sit where this
  // shape has its counters and tickets, and those must start at zero.
  TB200_CUDA_CHECK(cudaMemsetAsync(g_scratch_addr[dev], 0, L.counters_bytes, static_cast<cudaStream_t>(stream)));
  return tb200_gqa_decode(q, k, v, o, lse, real_seqlen_kv, uniform_seqlen, block_table, block_table_stride,
                          k_scale, v_scale, q_dtype, kv_dtype, o_dtype, batch, heads, heads_kv, dim, page_size,
                          kv_token_stride, kv_head_stride, kv_batch_stride, sm_scale, softcap, /*kv_pool_tokens=*/0,
                          /*flags=*/0, g_scratch_addr[dev], kDecodeStaticScratchBytes, stream);
}
