// Dense GQA prefill (flash-attention forward) for sm_100a: tcgen05 MMAs with TMEM accumulators,
// TMA-fed shared memory, online softmax in registers.
//
// Role in the reference: replaces GQAPrefillFwdKernel (src/tileops/kernels/attention/gqa_fwd.py:
// 309-468, 519-597 in tile-ai/TileOPs) and its Hopper-only warp-specialised variants
// (gqa_prefill_fwd_ws.py:59-433, gqa_fwd_ws.py:503-1030), none of which runs on sm_100.  Same
// math: S = Q K^T, bottom-right aligned causal mask, exp2-domain online softmax with fp32
// accumulation, O = P V, optional softcap, log2-domain LSE.
//
// One CTA = one 128-row Q tile of one (batch, q head); 6 warps:
//   warps 0-3  softmax / correction / epilogue: thread r owns row r (TMEM lane r), no shuffles
//   warp  4    TMA producer (one lane): Q once, then 64-key K_i and V_i tiles into 2-buffer rings
//   warp  5    MMA issuer (one lane) and TMEM allocator
// KV is consumed in tiles of 64 keys.  TMEM (256 columns per CTA): S0 [0,64) | S1 [64,128) |
// O [128,256); P_i (16-bit) overwrites the first 32 columns of S_i and feeds the second MMA
// straight from TMEM.  The MMA lane issues QK_0, QK_1, then PV_i, QK_{i+2} for i = 0, 1, ...:
// while the softmax warps work on S_i, the tensor core runs PV_{i-1} and QK_{i+1}, so inside one
// CTA the two sides overlap continuously.  TWO CTAs are resident per SM (97 KB of shared memory,
// 256 TMEM columns, at most 168 registers per thread each); the second one fills what is left and
// hides prologue and epilogue.  Every K/V buffer is refilled a full tile period before it is needed.
//
// Softmax is two passes over the S tile in TMEM (row max, then exp2 / sum / pack) to keep the
// register footprint small.  O in TMEM is rescaled only when some row of the warp saw its maximum
// grow by more than 2^8 since the value it is scaled to; until then the stale maximum is kept
// (P entries up to 256 are harmless in bf16 and fp32), and the final 1/l normalisation and the
// LSE use the same stale maximum, so the result is unchanged.
//
// Shared memory operands are [128 rows x 64 elements] panels (128-byte rows, 128B swizzle), two
// panels per 128x128 tile, written by TMA and described to the MMA by 64-bit matrix descriptors:
// Q and K are K-major (rows = M/N, 128 B = 64 K-elements), V is MN-major (rows = tokens = K).
//
// Every mbarrier wait is bounded; on a timeout the CTA records an error code, stops issuing work,
// lets its copies drain, frees its TMEM and returns.
#include <cuda_fp8.h>
#include <type_traits>

#include "gqa_prefill.cuh"

namespace tb200 {
namespace {

#ifndef TB200_PF_POLY
#define TB200_PF_POLY 0
#endif
#ifndef TB200_PF_TRUNC
#define TB200_PF_TRUNC 0
#endif
constexpr int kBM = 128;
constexpr int kBN = 64;                      // keys per S tile
constexpr int kStages = 2;                   // K, V and S buffers
constexpr int kQPanel = kBM * 128;           // 128 rows x 128 B (64 head dims)
constexpr int kKvPanel = kBN * 128;          // 64 rows x 128 B
constexpr int kThreads = 192;
constexpr int kThreadsF8 = 384;              // + warps 6, 7 idle and four converter warps 8-11 (e4m3 pages expanded in shared memory)
// Registers of the e4m3-page variant: 12 warps x 2 CTAs leave 80 per thread at launch; the softmax warpgroup
// takes 128 (setmaxnreg.inc) from what the other two warpgroups give back (setmaxnreg.dec to 56).  inc BLOCKS
// until the CTA's own pool - what it was launched with - holds that many, so the sums must fit the launch
// allocation; the host refuses the variant when the compiled kernel was given fewer than kF8LaunchRegs.
constexpr int kF8LaunchRegs = 80, kF8SoftmaxRegs = 128, kF8OtherRegs = 56;
static_assert(4 * kF8SoftmaxRegs + 8 * kF8OtherRegs <= 12 * kF8LaunchRegs, "setmaxnreg.inc would block forever");
// TMEM columns a CTA allocates: S0 | S1 | O = 64 + 64 + HD, rounded up to a power of two.  Head dims
// up to 128 leave room for two CTAs per SM (2 x 256 of 512 columns); 256 takes the whole TMEM.
__host__ __device__ constexpr uint32_t tmem_cols(int hd) { return hd <= 128 ? 256u : 512u; }
__host__ __device__ constexpr int ctas_per_sm(int hd) { return hd <= 128 ? 2 : 1; }
constexpr uint32_t kColS = 0, kColO = 128;    // S buffer s at columns [64 s, 64 s + 64)
#ifndef TB200_PF_F32X2
#define TB200_PF_F32X2 1
#endif
#ifndef TB200_PF_F8_CVT_CHUNKS
#define TB200_PF_F8_CVT_CHUNKS 4   // of a converter thread's four chunks, how many go through the XU pipe (4 measured fastest)
#endif

// Shared-memory plan for head dim HD (64 or 128): HD / 64 panels per operand tile.
template <int HD>
struct SmemLayoutT {
  static constexpr int kPanels = HD / 64;
  static constexpr int kQBytes = kPanels * kQPanel;    // 128 x HD 16-bit
  static constexpr int kKvBytes = kPanels * kKvPanel;  // 64 x HD 16-bit
  // offsets from the 1024-aligned base
  static constexpr int q = 0;
  static constexpr int k = q + kQBytes;
  static constexpr int v = k + kStages * kKvBytes;
  static constexpr int bars = v + kStages * kKvBytes;
  static constexpr int total = bars + 256;
};
// barrier indices
enum { B_QFULL = 0, B_KFULL = 1, B_KEMPTY = 3, B_VFULL = 5, B_VEMPTY = 7, B_SFULL = 9, B_PREADY = 11, B_ODONE = 13, B_OFINAL = 14, B_KRAW = 15, B_VRAW = 17, B_COUNT = 19 };

// Optional timeline for tuning (-DTB200_TRACE): CTA kTraceCta stamps %globaltimer-free clock64()
// values of its MMA lane (slots 0-3) and of softmax thread 0 (slots 4-8) for the first
// kTraceIters KV tiles into the workspace behind the status word.
#ifdef TB200_TRACE
constexpr int kTraceIters = 64, kTraceSlots = 10, kTraceCta = 600;
#define TB200_STAMP(slot, j)                                                                          \
  do {                                                                                                \
    if (blockIdx.x == kTraceCta && (j) < kTraceIters)                                                 \
      reinterpret_cast<long long*>(p.status + 64)[(j) * kTraceSlots + (slot)] = clock64();            \
  } while (0)
#else
#define TB200_STAMP(slot, j) do {} while (0)
#endif

// ---- PTX wrappers: tb200_async.cuh (mbarrier, TMA) and tb200_tcgen05.cuh (MMA, TMEM) ----------------
// Bounded wait.  Returns false when the CTA is aborting (this wait ran out, or another role's did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
  return mbar_wait_bounded(bar, parity, abort_flag, status, code, kWaitCycles);
}

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float lo, float hi) { return pack2<T>(lo, hi); }

// ---- kernel --------------------------------------------------------------------------------
// kPaged = false: dense [batch, seq, heads, HD] tensors, one KV segment.
// kPaged = true: requests packed along the row dimension (cu_q), and two KV segments per request:
// the tokens already in the paged cache (read through the block table with map_kp / map_vp, all
// visible to every query row) and then the request's own new tokens (read from k_new / v_new with
// map_k / map_v, causal inside the chunk).  CTAs of the first q head of a KV group also copy their
// 128 new K/V rows into the pages; attention never reads those copies, so no CTA waits for another.
//
// kF8 (with kPaged, head dim 128): the pages hold e4m3 with one fp32 scale per tensor.  A cached tile arrives as
// 64 rows of 128 bytes in the SECOND panel's place of its 16 KB buffer; two converter warps (warps 6, 7; thread =
// row) expand it in place to the 16-bit, 128B-swizzled two-panel tile the MMA descriptors expect (x = float(x8) *
// scale rounded to T, the reference's dequantisation): a thread reads its whole source row into registers first,
// then writes panel 0 (nobody's source) and panel 1 (its own source row), so no thread overwrites what another
// still has to read.  K/V "full" barriers then take two arrivals: the converter warps' for a cached tile, the
// producer's arrive + arrive.expect_tx for a 16-bit tile of the chunk.  The appended rows are quantised
// (e4m3(x / scale), saturating) by the appending CTAs.
template <typename T, bool kSoftcap, int HD, bool kPaged, bool kF8 = false>
__global__ void __launch_bounds__(kF8 ? kThreadsF8 : kThreads, ctas_per_sm(HD))
gqa_prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_kp,
                   const __grid_constant__ CUtensorMap map_vp, PrefillParams p) {
  static_assert(!kF8 || (kPaged && HD == 128), "the e4m3-page variant serves the paged kernel at head dim 128");
  using SmemLayout = SmemLayoutT<HD>;
  constexpr int kHD = HD;
  constexpr int kQBytes = SmemLayout::kQBytes, kKvBytes = SmemLayout::kKvBytes;
  constexpr uint32_t kTmemCols = tmem_cols(HD);
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SmemLayout::bars);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  // an earlier CTA of this launch gave up on a wait: do not start more work (one thread reads
  // the flag so that the whole CTA takes the same decision)
  __shared__ int s_skip;
  if (tid == 0) s_skip = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_skip != 0) return;

  // ---- which tile ---------------------------------------------------------------------
  const int n_m = (p.seqlen_q + kBM - 1) / kBM;            // paged: seqlen_q is the longest request
  const int per_m = p.heads * p.batch;
  const int mt = n_m - 1 - int(blockIdx.x) / per_m;        // heaviest (last) row tiles first
  const int rest = int(blockIdx.x) % per_m;
  const int b = rest / p.heads, h = rest % p.heads;
  const int hk = h / (p.heads / p.heads_kv);
  const int m0 = mt * kBM;
  // rows of this tile in the q / o tensors, and where the (new) K/V segment starts
  int q_row0 = m0, q_batch = b, q_len = p.seqlen_q, kv_len = p.seqlen_kv, old_len = 0;
  int kv_row0 = 0;                                         // row of the (new) segment's first key
  if (kPaged) {
    const int q0 = p.cu_q[b];
    q_len = p.cu_q[b + 1] - q0;
    if (m0 >= q_len) return;                               // the whole CTA: nothing allocated yet
    kv_row0 = p.cu_kv ? p.cu_kv[b] : q0;
    kv_len = p.cu_kv ? p.cu_kv[b + 1] - kv_row0 : q_len;
    old_len = p.cache_lens ? p.cache_lens[b] : 0;
    q_row0 = q0 + m0;
    q_batch = 0;
  }
  const int off = kv_len - q_len;                          // bottom-right alignment (0 when paged)
  const int n_old = (old_len + kBN - 1) / kBN;             // tiles of cached tokens (0 when dense)
  // Row i sees keys j with i + off - win_left <= j <= i + off + up_extra (each bound only if it
  // applies): causal means up_extra = 0, otherwise the right window.
  const bool has_upper = p.is_causal || p.win_right >= 0;
  const int up_extra = p.is_causal ? 0 : p.win_right;
  int n_end = (kv_len + kBN - 1) / kBN;                    // one past the last tile of the new segment
  if (has_upper) {
    const long long last_key = (long long)m0 + kBM - 1 + off + up_extra;   // of the tile's last row
    n_end = last_key < 0 ? 0 : int(min((long long)n_end, last_key / kBN + 1));
  }
  int tile0 = 0;                                           // first tile any row of this CTA can see
  if (p.win_left >= 0) tile0 = max(0, m0 + off - p.win_left) / kBN;
  const int n_new = max(0, n_end - tile0);
  const int n_kv = n_old + n_new;

  if (tid == 0) {
    mbar_init(bar(B_QFULL), 1);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(bar(B_KFULL + s), kF8 ? 4 : 1);
      mbar_init(bar(B_KEMPTY + s), 1);
      mbar_init(bar(B_VFULL + s), kF8 ? 4 : 1);
      mbar_init(bar(B_VEMPTY + s), 1);
      mbar_init(bar(B_KRAW + s), 1);
      mbar_init(bar(B_VRAW + s), 1);
      mbar_init(bar(B_SFULL + s), 1);
      mbar_init(bar(B_PREADY + s), 128);
    }
    mbar_init(bar(B_ODONE), 1);
    mbar_init(bar(B_OFINAL), 1);
    *s_abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(kTmemCols));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t idesc_qk = make_idesc(fmt, 0, kBN);
  constexpr uint32_t idesc_pv = make_idesc(fmt, 1, kHD);

  if (n_kv > 0) {
   if (warp >= 4) {
    // (kF8) the warpgroups of the single-lane roles and of the converters give registers back; the role code is
    // nested under the instruction so that the compiler allocates each side for what it was given
    if constexpr (kF8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kF8OtherRegs));
    if (warp == 4) {
      // ================= TMA producer =================
      if (lane == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
        if (kPaged && n_old > 0) {
          asm volatile("prefetch.tensormap [%0];" ::"l"(&map_kp) : "memory");
          asm volatile("prefetch.tensormap [%0];" ::"l"(&map_vp) : "memory");
        }
        mbar_expect_tx(bar(B_QFULL), kQBytes);
#pragma unroll
        for (int pn = 0; pn < kHD / 64; ++pn)
          tma_load_4d(sbase + SmemLayout::q + pn * kQPanel, &map_q, bar(B_QFULL), pn * 64, h, q_row0, q_batch);
        // one 64-key tile of K or V: HD / 64 panels; a cached tile is gathered page by page
        // (page_box rows per copy) through the block table.  The pool rows of a tile's copies are
        // looked up once for K and V together, one tile ahead, so that the block-table read never
        // sits between a freed stage and its refill.
        constexpr int kMaxBoxes = kBN / 16;                  // the smallest page holds 16 tokens
        int rows_cur[kMaxBoxes], rows_next[kMaxBoxes];
        auto lookup = [&](int i, int (&rows)[kMaxBoxes]) {
          if (!(kPaged && i < n_old)) return;
#pragma unroll
          for (int x = 0; x < kMaxBoxes; ++x) {
            const int r = x * p.page_box;
            if (r < kBN) {
              // the last cached tile may reach past old_len: look up the page of a live token there (the
              // rows are masked and their V cleared), never an entry behind the request's pages
              const int tok = min(i * kBN + r, old_len - 1);
              const int page = p.bt[(long long)b * p.bt_stride + (tok >> p.page_shift)];
              rows[x] = page * p.page_size + ((i * kBN + r) & (p.page_size - 1));
            }
          }
        };
        auto load_tile = [&](uint32_t dst, uint32_t full_bar, const CUtensorMap* dense_map,
                             const CUtensorMap* pool_map, int i, const int (&rows)[kMaxBoxes]) {
          if (kPaged && i < n_old) {
#pragma unroll
            for (int x = 0; x < kMaxBoxes; ++x) {
              const int r = x * p.page_box;
              if (r < kBN) {
                if constexpr (kF8) {
                  // e4m3 rows (128 bytes each) into the second panel's place; the converter warps expand them
                  tma_load_4d(dst + kKvPanel + r * 128, pool_map, full_bar, 0, hk, rows[x], 0);
                } else {
#pragma unroll
                  for (int pn = 0; pn < kHD / 64; ++pn)
                    tma_load_4d(dst + pn * kKvPanel + r * 128, pool_map, full_bar, pn * 64, hk, rows[x], 0);
                }
              }
            }
          } else {
            const int row = kv_row0 + (tile0 + i - n_old) * kBN;
#pragma unroll
            for (int pn = 0; pn < kHD / 64; ++pn)
              tma_load_4d(dst + pn * kKvPanel, dense_map, full_bar, pn * 64, hk, row, q_batch);
          }
        };
        lookup(0, rows_cur);
        for (int i = 0; i < n_kv; ++i) {
          const int s = i & 1;
          const uint32_t par = (i >> 1) & 1;
          if (i + 1 < n_kv) lookup(i + 1, rows_next);         // in flight during the waits below
          const bool raw = kF8 && i < n_old;                  // an e4m3 tile: half the bytes, handed to the converter warps
          const uint32_t k_bar = raw ? bar(B_KRAW + s) : bar(B_KFULL + s);
          const uint32_t v_bar = raw ? bar(B_VRAW + s) : bar(B_VFULL + s);
          if (!mbar_wait(bar(B_KEMPTY + s), par ^ 1, s_abort, p.status, 101)) break;
          if (kF8 && !raw) { mbar_arrive(k_bar); mbar_arrive(k_bar); mbar_arrive(k_bar); }   // "full" takes four arrivals here
          mbar_expect_tx(k_bar, raw ? kKvBytes / 2 : kKvBytes);
          load_tile(sbase + SmemLayout::k + s * kKvBytes, k_bar, &map_k, &map_kp, i, rows_cur);
          if (!mbar_wait(bar(B_VEMPTY + s), par ^ 1, s_abort, p.status, 102)) break;
          if (kF8 && !raw) { mbar_arrive(v_bar); mbar_arrive(v_bar); mbar_arrive(v_bar); }
          mbar_expect_tx(v_bar, raw ? kKvBytes / 2 : kKvBytes);
          load_tile(sbase + SmemLayout::v + s * kKvBytes, v_bar, &map_v, &map_vp, i, rows_cur);
#pragma unroll
          for (int x = 0; x < kMaxBoxes; ++x) rows_cur[x] = rows_next[x];
        }
      }
    } else if (warp == 5) {
      // ================= MMA issuer =================
      if (lane == 0) {
        bool ok = mbar_wait(bar(B_QFULL), 0, s_abort, p.status, 201);
        // The buffers are fixed, so the matrix descriptors are built once; a k-step only adds
        // its byte offset (>> 4) to the start-address field.
        const uint64_t dq = make_desc(sbase + SmemLayout::q, 16, 1024);
        const uint64_t dk0 = make_desc(sbase + SmemLayout::k, 16, 1024);
        const uint64_t dv0 = make_desc(sbase + SmemLayout::v, kKvPanel, 1024);
        constexpr uint64_t kBufStep = kKvBytes >> 4;        // second buffer, in start-address units
        // S_i = Q K_i^T into S buffer i&1.  It overwrites P_{i-2}, which PV_{i-2} (issued
        // earlier by this thread) reads: the tensor core runs one thread's MMAs in issue order.
        auto issue_qk = [&](int i) -> bool {
          const int s = i & 1;
          if (!mbar_wait(bar(B_KFULL + s), (i >> 1) & 1, s_abort, p.status, 202)) return false;
          TB200_STAMP(0, i);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kHD / 16; ++ks) {
            // K-major operands: 16 elements per step = 32 B inside the 128 B swizzled row; after 4
            // steps move to the second 64-element panel (16 KB further for Q, 8 KB for K)
            const uint32_t oq = ((ks >> 2) * kQPanel + (ks & 3) * 32) >> 4;
            const uint32_t ok_ = ((ks >> 2) * kKvPanel + (ks & 3) * 32) >> 4;
            tc_mma_ss(tmem + kColS + s * kBN, dq + oq, dk0 + s * kBufStep + ok_, idesc_qk, ks > 0 ? 1u : 0u);
          }
          tc_commit(bar(B_SFULL + s));
          tc_commit(bar(B_KEMPTY + s));
          TB200_STAMP(1, i);
          return true;
        };
        if (ok) ok = issue_qk(0);
        if (ok && n_kv > 1) ok = issue_qk(1);
        for (int i = 0; ok && i < n_kv; ++i) {
          const int s = i & 1;
          const uint32_t par = (i >> 1) & 1;
          if (!mbar_wait(bar(B_VFULL + s), par, s_abort, p.status, 203)) break;
          if (!mbar_wait(bar(B_PREADY + s), par, s_abort, p.status, 204)) break;
          TB200_STAMP(2, i);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kBN / 16; ++ks) {
            // B = V: MN-major, 16 tokens per step = 16 rows of 128 B; the two 64-wide d panels
            // are kKvPanel apart (leading offset), 8-row groups 1024 B apart (stride offset)
            tc_mma_ts(tmem + kColO, tmem + kColS + s * kBN + ks * 8, dv0 + s * kBufStep + ((ks * 2048) >> 4), idesc_pv,
                      (i > 0 || ks > 0) ? 1u : 0u);
          }
          tc_commit(bar(B_VEMPTY + s));
          tc_commit(bar(B_ODONE));
          if (i == n_kv - 1) tc_commit(bar(B_OFINAL));   // its own barrier: B_ODONE may be two phases ahead of a late reader
          TB200_STAMP(3, i);
          if (i + 2 < n_kv) ok = issue_qk(i + 2);
        }
      }
    } else if (warp >= 6) {
      // ================= converter warps 8-11 (kF8): expand e4m3 tiles in place; warps 6, 7 only fill their warpgroup =================
      if constexpr (kF8) {
       if (warp >= 8) {
        const int r = (tid - 256) >> 1;                      // row of the tile, 0..63; two threads per row
        const int c0 = ((tid - 256) & 1) * 4;                // this thread's four 16-byte source chunks
        // Exact expansion e4m3 -> T (every e4m3 value is a T value); the tensors' scalar scales are applied by
        // the softmax threads (K: in the score scale of cached tiles; V: in the exponent of P), which costs
        // them nothing per element.  Two ways to expand a byte pair, both exact, on different pipes:
        //   * cvt.rn.f16x2.e4m3x2 (XU pipe, which the exponentials of the softmax warps on the same scheduler
        //     need; for bf16 followed by two f16 -> f32 conversions and a byte permute that takes the high halves);
        //   * integer: the bytes go to the high byte of each half, the 7 magnitude bits move down to T's
        //     exponent/mantissa boundary, which gives a T number whose exponent bias is off by 2^8 (f16) or
        //     2^120 (bf16), subnormals included, and one exact multiply corrects it (5 instructions per pair).
        // Measured on 8 x 512 new tokens over 8 x 4096 cached (fp16 / bf16; the same shape with a 16-bit cache
        // takes 363 us, the three-launch path - gather, packed prefill, append - 430 us): two converter warps with
        // cvt 496 us (their two schedulers XU bound), with the integer path 752 us (issue bound); four warps, one
        // per scheduler: cvt 518 / 554 us, half and half 562 / 588 us, integer 613 / 616 us.  Every variant loses to
        // the separate gather: each of the 16 CTAs that share a (request, KV head) converts the same tile again,
        // on schedulers whose issue slots and XU pipe the softmax already fills, while the gather kernel converts
        // every byte once at HBM speed.  The variant therefore stays opt-in; what it saves is memory (no packed
        // 16-bit copy of the cache).
        constexpr int kCvtChunks = TB200_PF_F8_CVT_CHUNKS;
        auto expand = [&](unsigned char* tile) {
          const int sw = r & 7;
          uint4 raw[4];
#pragma unroll
          for (int c = 0; c < 4; ++c) raw[c] = *reinterpret_cast<const uint4*>(tile + kKvPanel + r * 128 + (((c0 + c) ^ sw) << 4));
          __syncwarp();      // the row's other thread (the neighbouring lane) has its source too: the row may be overwritten
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int c = c0 + cc;
            const uint32_t w[4] = {raw[cc].x, raw[cc].y, raw[cc].z, raw[cc].w};
            uint32_t o16[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (cc < kCvtChunks) {
                uint32_t h;
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h) : "h"(uint16_t(w[j >> 1] >> ((j & 1) * 16))));
                if constexpr (std::is_same<T, __half>::value) {
                  o16[j] = h;
                } else {
                  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
                  o16[j] = __byte_perm(__float_as_uint(f.x), __float_as_uint(f.y), 0x7632);
                }
              } else {
                const uint32_t x = (j & 1) ? __byte_perm(w[j >> 1], 0u, 0x3424) : __byte_perm(w[j >> 1], 0u, 0x1404);
                if constexpr (std::is_same<T, __half>::value) {
                  const uint32_t t = (x & 0x80008000u) | ((x >> 1) & 0x3f803f80u);
                  asm("mul.rn.f16x2 %0, %1, %2;\n" : "=r"(o16[j]) : "r"(t), "r"(0x5c005c00u));        // x 2^8
                } else {
                  const uint32_t t = (x & 0x80008000u) | ((x >> 4) & 0x07f007f0u);
                  asm("mul.rn.bf16x2 %0, %1, %2;\n" : "=r"(o16[j]) : "r"(t), "r"(0x7b807b80u));      // x 2^120
                }
              }
            }
            // 16 source elements = output chunks 2c and 2c + 1 of the 256-byte row: panel c / 4, chunks (2c) % 8, + 1
            unsigned char* orow = tile + (c >> 2) * kKvPanel + r * 128;
            *reinterpret_cast<uint4*>(orow + ((((2 * c) & 7) ^ sw) << 4)) = make_uint4(o16[0], o16[1], o16[2], o16[3]);
            *reinterpret_cast<uint4*>(orow + ((((2 * c + 1) & 7) ^ sw) << 4)) = make_uint4(o16[4], o16[5], o16[6], o16[7]);
          }
          // every lane makes its own stores visible (CTA scope, then to the async proxy) before lane 0 arrives for the warp
          __threadfence_block();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        };
        for (int i = 0; i < n_old; ++i) {
          const int s = i & 1;
          const uint32_t par = (i >> 1) & 1;
          if (!__all_sync(0xffffffffu, mbar_wait(bar(B_KRAW + s), par, s_abort, p.status, 401))) break;
          expand(smem + SmemLayout::k + s * kKvBytes);
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_KFULL + s));
          if (!__all_sync(0xffffffffu, mbar_wait(bar(B_VRAW + s), par, s_abort, p.status, 402))) break;
          expand(smem + SmemLayout::v + s * kKvBytes);
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_VFULL + s));
        }
       }
      }
    }
   } else {
    {
      if constexpr (kF8) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kF8SoftmaxRegs));
      // ================= softmax / correction / epilogue (thread = row) =================
      const int row = tid;                                  // 0..127 == TMEM lane
      const uint32_t lane_addr = uint32_t(warp * 32) << 16;
      const float cap = p.softcap;
      const float c = kSoftcap ? kLog2e : p.sm_scale * kLog2e;   // multiplies the raw (or capped) score
      const float pre = kSoftcap ? p.sm_scale / cap : 0.f;
      const int q_idx = m0 + row;                           // row inside its batch element / request
      const int causal_limit = has_upper ? q_idx + off + up_extra : 0x7fffffff;  // last visible key of this row
      const int key_floor = p.win_left >= 0 ? q_idx + off - p.win_left : int(0x80000000);  // first visible key
      int key_limit = causal_limit, seg_len = kv_len;       // of the segment the current tile belongs to

      if (kPaged && p.k_pages != nullptr && h % (p.heads / p.heads_kv) == 0) {
        // Append this tile's new K/V rows of KV head hk to the pages.  16 bytes per thread and step;
        // consecutive threads cover one row, so loads and stores are coalesced.
        constexpr int kChunks = kHD * 2 / 16;
        const int rows = min(kBM, q_len - m0);
        const size_t row_bytes = size_t(p.heads_kv) * kHD * 2;
        for (int idx = tid; idx < rows * kChunks; idx += 128) {
          const int r = idx / kChunks, ch = idx % kChunks;
          const int pos = old_len + m0 + r;
          const int page = p.bt[(long long)b * p.bt_stride + (pos >> p.page_shift)];
          const size_t dst_row = size_t(page) * p.page_size + (pos & (p.page_size - 1));
          const size_t src = size_t(q_row0 + r) * row_bytes + size_t(hk) * kHD * 2 + ch * 16;
          const uint4 kk = *reinterpret_cast<const uint4*>(static_cast<const char*>(p.k_new) + src);
          const uint4 vv = *reinterpret_cast<const uint4*>(static_cast<const char*>(p.v_new) + src);
          if constexpr (kF8) {
            // 8 elements -> 8 bytes: e4m3(x / scale), round to nearest even, saturating
            const size_t dst = (dst_row * p.heads_kv + hk) * kHD + ch * 8;
            const float ks = *p.k_scale, vs = *p.v_scale;
            auto quant = [](const uint4& x, float scale) {
              const uint32_t w[4] = {x.x, x.y, x.z, x.w};
              uint32_t out[2] = {0u, 0u};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = unpack2<T>(w[j]);
                const uint32_t b0 = __nv_cvt_float_to_fp8(__fdiv_rn(f.x, scale), __NV_SATFINITE, __NV_E4M3);
                const uint32_t b1 = __nv_cvt_float_to_fp8(__fdiv_rn(f.y, scale), __NV_SATFINITE, __NV_E4M3);
                out[j >> 1] |= (b0 | (b1 << 8)) << ((j & 1) * 16);
              }
              return make_uint2(out[0], out[1]);
            };
            *reinterpret_cast<uint2*>(static_cast<unsigned char*>(p.k_pages) + dst) = quant(kk, ks);
            *reinterpret_cast<uint2*>(static_cast<unsigned char*>(p.v_pages) + dst) = quant(vv, vs);
          } else {
            const size_t dst = dst_row * row_bytes + size_t(hk) * kHD * 2 + ch * 16;
            *reinterpret_cast<uint4*>(static_cast<char*>(p.k_pages) + dst) = kk;
            *reinterpret_cast<uint4*>(static_cast<char*>(p.v_pages) + dst) = vv;
          }
        }
      }
      const uint32_t s_addr0 = tmem + lane_addr + kColS;
      const uint32_t o_addr = tmem + lane_addr + kColO;
      float m_run = -INFINITY, l_run = 0.f;   // m_run: the maximum O and l are currently scaled to
      // e4m3 pages (kF8): the cached tiles hold the bare e4m3 values.  K's scalar scale multiplies their raw scores
      // (and their maximum, to keep one running maximum in the units of the chunk's own tiles); V's is added, as
      // log2, to the exponent of their P, so that P V comes out scaled, and their row sums are kept apart
      // (l_cached, in units of v_scale) and divided by v_scale at the end.
      float l_cached = 0.f, pre_t = pre;
      const float k_sc = kF8 ? *p.k_scale : 1.f, v_sc = kF8 ? *p.v_scale : 1.f;
      const float log2_v_sc = kF8 ? log2f(v_sc) : 0.f;
      constexpr bool kBf16 = TB200_PF_TRUNC && std::is_same<T, __nv_bfloat16>::value;
      constexpr float kTruncFix = kBf16 ? 0.0028150156f : 0.f;   // log2(1 + 2^-9)
      bool ok = true;

      // transform of one loaded chunk: softcap and mask (only on tiles that need it)
      auto prepare = [&](uint32_t (&r)[32], int key0, bool need_mask) {
        if (kSoftcap) {
#pragma unroll
          for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(cap * fast_tanh(__uint_as_float(r[e]) * pre_t));
        }
        if (need_mask) {
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            const int key = key0 + e;
            if (key > key_limit || key < key_floor || key >= seg_len) r[e] = 0xff800000u;   // -inf
          }
        }
      };

      for (int j = 0; j < n_kv; ++j) {
        const int sb = j & 1;                               // S / P buffer of this tile
        const uint32_t s_addr = s_addr0 + sb * kBN;
        // the warp leaves the loop together: the TMEM loads below are warp-collective
        if (!__all_sync(0xffffffffu, mbar_wait(bar(B_SFULL + sb), (j >> 1) & 1, s_abort, p.status, 301))) { ok = false; break; }
        tc_fence_after();
        if (tid == 0) TB200_STAMP(4, j);
        int k0 = j * kBN;                                   // first key of the tile inside its segment
        const bool scaled_tile = kF8 && j < n_old;          // a cached tile of bare e4m3 values
        if (kF8 && kSoftcap) pre_t = scaled_tile ? pre * k_sc : pre;
        bool need_mask;
        if (kPaged && j < n_old) {
          key_limit = 0x7fffffff; seg_len = old_len;        // cached tokens: visible to every row
          need_mask = k0 + kBN > old_len;
        } else {
          k0 += (tile0 - n_old) * kBN;
          key_limit = causal_limit; seg_len = kv_len;
          need_mask = (has_upper && k0 + kBN - 1 > m0 + off + up_extra) || (k0 + kBN > kv_len) ||
                      (p.win_left >= 0 && k0 < m0 + kBM - 1 + off - p.win_left);
        }

        // ---- pass 1: row maximum.  TMEM loads are asynchronous: the next 32 columns are in flight
        // while the maximum of the current 32 is taken. ----
        uint32_t r0[32], r1[32];
        auto chunk_max = [&](uint32_t (&r)[32], int cgi, float mx_in) {
          prepare(r, k0 + cgi * 32, need_mask);
          float a = mx_in, bb = -INFINITY;
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            a = max3(a, __uint_as_float(r[e]), __uint_as_float(r[e + 1]));
            bb = max3(bb, __uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
          }
          return fmaxf(a, bb);
        };
        float mx = -INFINITY;
        tc_ld32(s_addr, r0);
        tc_wait_ld(r0);
        tc_ld32(s_addr + 32, r1);
        mx = chunk_max(r0, 0, mx);
        tc_wait_ld(r1);
        tc_ld32(s_addr, r0);          // first chunk of pass 2, in flight during the decision below
        mx = chunk_max(r1, 1, mx);
        if (kF8 && !kSoftcap && scaled_tile) mx *= k_sc;    // raw maxima of cached tiles -> units of the chunk's tiles

        if (tid == 0) TB200_STAMP(5, j);
        // ---- decide whether the running maximum moves (and O has to be rescaled) ----
        const float m_new = fmaxf(m_run, mx);
        const bool grow = (m_new - m_run) * c > kRescaleThreshold || (m_run == -INFINITY && m_new != -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          // 1 for a row that still has seen no key (avoids inf - inf), 0 for a row seeing its first
          const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2((m_run - m_new) * c);
          l_run *= alpha;
          l_cached *= alpha;
          if (j > 0) {
            // PV_{j-1} was issued after QK_j and may still be adding into O: wait for it.  (It
            // depends only on P_{j-1}, which these warps handed over a tile ago.)
            if (!__all_sync(0xffffffffu, mbar_wait(bar(B_ODONE), (j - 1) & 1, s_abort, p.status, 302))) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int cgi = 0; cgi < kHD / 32; ++cgi) {
              uint32_t ov[32];
              tc_ld32(o_addr + cgi * 32, ov);
              tc_wait_ld(ov);
#pragma unroll
              for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
              tc_st32(o_addr + cgi * 32, ov);
            }
          }
          m_run = m_new;
        }
        if (tid == 0) TB200_STAMP(6, j);
        const float neg_mc = ((m_run == -INFINITY) ? 0.f : -m_run * c) + kTruncFix + (scaled_tile ? log2_v_sc : 0.f);
        const float ck = (kF8 && !kSoftcap && scaled_tile) ? c * k_sc : c;   // multiplier of this tile's raw scores

        // ---- pass 2: p = 2^(s*c - m*c), row sum, P (16-bit) over the first 64 columns of S ----
        float lsum0 = 0.f, lsum1 = 0.f;
#if TB200_PF_F32X2
        uint64_t lsum_a = 0, lsum_b = 0;                    // two (even key, odd key) pairs of partial sums
        const uint64_t c2 = f2_pack(ck, ck), neg_mc2 = f2_pack(neg_mc, neg_mc);
#endif
        // Two tuning switches, both off: they measured slower or neutral on B200 (this pass is
        // bound by instruction latency, not by the MUFU pipe).  TB200_PF_POLY evaluates every second
        // exponential on the FMA pipe on tiles without masked entries.  TB200_PF_TRUNC packs bf16 P
        // by taking the high halves of the two floats with one PRMT; kTruncFix in the exponent
        // scales p by (1 + 2^-9) first, which turns truncation into round-to-nearest on average
        // (the row sum carries the same factor, so O = (P V) / l is unaffected; the LSE subtracts it).
        auto chunk_exp = [&](uint32_t (&r)[32], int cgi, auto masked) {
          constexpr bool kMasked = decltype(masked)::value;
          prepare(r, k0 + cgi * 32, need_mask);
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
#if TB200_PF_F32X2
            float x0, x1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1])), c2, neg_mc2), x0, x1);
            const float p0 = fast_exp2(x0);
            const float p1 = fast_exp2(x1);
            if (e & 1) lsum_b = f2_add(lsum_b, f2_pack(p0, p1)); else lsum_a = f2_add(lsum_a, f2_pack(p0, p1));
#else
            const float x0 = fmaf(__uint_as_float(r[2 * e]), ck, neg_mc);
            const float x1 = fmaf(__uint_as_float(r[2 * e + 1]), ck, neg_mc);
            const float p0 = fast_exp2(x0);
            const float p1 = (kMasked || !TB200_PF_POLY) ? fast_exp2(x1) : exp2_poly(x1);
            lsum0 += p0;
            lsum1 += p1;
#endif
            if constexpr (kBf16)
              pk[e] = prmt(__float_as_uint(p0), __float_as_uint(p1), 0x7632);
            else
              pk[e] = pack_pair<T>(p0, p1);
          }
          // P chunk cgi lands in columns [16 cgi, 16 cgi + 16): inside S chunks already consumed,
          // and below the chunk that is being loaded
          tc_st16(s_addr + cgi * 16, pk);
        };
        auto pass2 = [&](auto masked) {
          tc_wait_ld(r0);
          tc_ld32(s_addr + 32, r1);
          chunk_exp(r0, 0, masked);
          tc_wait_ld(r1);
          chunk_exp(r1, 1, masked);
        };
        if (need_mask) pass2(std::true_type{}); else pass2(std::false_type{});
#if TB200_PF_F32X2
        f2_unpack(f2_add(lsum_a, lsum_b), lsum0, lsum1);
#endif
        if (scaled_tile) l_cached += lsum0 + lsum1; else l_run += lsum0 + lsum1;
        if (tid == 0) TB200_STAMP(7, j);
        if (kPaged && k0 + kBN > seg_len) {
          // Ragged last tile of a segment: the V rows behind it are another request's tokens or
          // unwritten page memory.  Their P is zero, but 0 x NaN is NaN, so clear them before the
          // MMA reads the tile (whole 128-byte rows: the swizzle permutes only inside a row).
          if (!__all_sync(0xffffffffu, mbar_wait(bar(B_VFULL + sb), (j >> 1) & 1, s_abort, p.status, 304))) { ok = false; break; }
          const int first = seg_len - k0;                   // 1 .. 63 valid rows
          unsigned char* vt = smem + SmemLayout::v + sb * kKvBytes;
          constexpr int kRowChunks = 128 / 16;
          for (int idx = tid; idx < (kBN - first) * kRowChunks * (kHD / 64); idx += 128) {
            const int pn = idx / ((kBN - first) * kRowChunks);
            const int rem = idx % ((kBN - first) * kRowChunks);
            *reinterpret_cast<uint4*>(vt + pn * kKvPanel + (first + rem / kRowChunks) * 128 + (rem % kRowChunks) * 16) =
                make_uint4(0, 0, 0, 0);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(B_PREADY + sb));
        if (tid == 0) TB200_STAMP(8, j);
      }

      // ---- epilogue: O / l -> global, LSE ----
      if (ok) ok = mbar_wait(bar(B_OFINAL), 0, s_abort, p.status, 303);
      ok = __all_sync(0xffffffffu, ok);
      if (kF8) l_run += l_cached / v_sc;
      if (ok) {
        tc_fence_after();
        const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
        T* orow = reinterpret_cast<T*>(p.o) +
                  ((kPaged ? size_t(q_row0 + row) : size_t(b) * p.seqlen_q + q_idx) * p.heads + h) * kHD;
#pragma unroll
        for (int cgi = 0; cgi < kHD / 32; ++cgi) {
          uint32_t ov[32];
          tc_ld32(o_addr + cgi * 32, ov);
          tc_wait_ld(ov);
          if (q_idx < q_len) {
#pragma unroll
            for (int e = 0; e < 32; e += 8) {
              uint4 w;
              w.x = pack_pair<T>(__uint_as_float(ov[e]) * inv_l, __uint_as_float(ov[e + 1]) * inv_l);
              w.y = pack_pair<T>(__uint_as_float(ov[e + 2]) * inv_l, __uint_as_float(ov[e + 3]) * inv_l);
              w.z = pack_pair<T>(__uint_as_float(ov[e + 4]) * inv_l, __uint_as_float(ov[e + 5]) * inv_l);
              w.w = pack_pair<T>(__uint_as_float(ov[e + 6]) * inv_l, __uint_as_float(ov[e + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + cgi * 32 + e) = w;
            }
          }
        }
        if (p.lse && q_idx < q_len)   // [batch, heads, seqlen_q], or [heads, total_q] for packed requests
          p.lse[kPaged ? size_t(h) * p.total_q + q_row0 + row : (size_t(b) * p.heads + h) * p.seqlen_q + q_idx] =
              l_run > 0.f ? m_run * c + log2f(l_run) - kTruncFix : -INFINITY;
      }
    }
   }
  } else if (warp < 4) {
    // the whole row tile is masked: zeros, LSE = -inf
    const int q_idx = m0 + tid;
    if (q_idx < q_len) {
      T* orow = reinterpret_cast<T*>(p.o) +
                ((kPaged ? size_t(q_row0 + tid) : size_t(b) * p.seqlen_q + q_idx) * p.heads + h) * kHD;
      const uint4 z = make_uint4(0, 0, 0, 0);
      for (int e = 0; e < kHD; e += 8) *reinterpret_cast<uint4*>(orow + e) = z;
      if (p.lse)
        p.lse[kPaged ? size_t(h) * p.total_q + q_row0 + tid : (size_t(b) * p.heads + h) * p.seqlen_q + q_idx] = -INFINITY;
    }
  }

  // ---- teardown -----------------------------------------------------------------------
  __syncwarp();   // the single-lane roles rejoin their warps before the block-wide barrier
  tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    // give copies still in flight time to land before the shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  if (warp == 5) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
  }
}

// ---- host side ------------------------------------------------------------------------------

template <typename T, bool kSoftcap, int HD, bool kPaged, bool kF8 = false>
int launch_prefill(const PrefillMaps& m, const PrefillParams& p, cudaStream_t stream) {
  auto kern = gqa_prefill_kernel<T, kSoftcap, HD, kPaged, kF8>;
  const int smem = SmemLayoutT<HD>::total + 1024;
  if constexpr (kF8) {
    // the softmax warpgroup's setmaxnreg.inc can only be served from the registers the CTA was launched with
    static thread_local int launch_regs = -1;
    if (launch_regs < 0) {
      cudaFuncAttributes attr;
      TB200_CUDA_CHECK(cudaFuncGetAttributes(&attr, kern));
      launch_regs = attr.numRegs;
    }
    if (launch_regs < kF8LaunchRegs)
      TB200_FAIL(TB200_ERR_UNSUPPORTED, "the e4m3-page prefill kernel was compiled with %d registers per thread, %d needed",
                 launch_regs, kF8LaunchRegs);
  }
  static thread_local bool configured[64] = {false};       // per device, for this instantiation
  int dev = 0;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    TB200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  const int n_m = (p.seqlen_q + kBM - 1) / kBM;
  const long long grid = (long long)n_m * p.heads * p.batch;
  if (grid > 0x7fffffffLL) TB200_FAIL(TB200_ERR_UNSUPPORTED, "problem too large for one launch");
  kern<<<unsigned(grid), kF8 ? kThreadsF8 : kThreads, smem, stream>>>(m.q, m.k, m.v, m.kp, m.vp, p);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}

template <int HD, bool kPaged>
int dispatch_prefill(int dtype, const PrefillMaps& m, const PrefillParams& p, cudaStream_t s) {
  if (p.softcap > 0.f)
    return dtype == TB200_BF16 ? launch_prefill<__nv_bfloat16, true, HD, kPaged>(m, p, s)
                               : launch_prefill<__half, true, HD, kPaged>(m, p, s);
  return dtype == TB200_BF16 ? launch_prefill<__nv_bfloat16, false, HD, kPaged>(m, p, s)
                             : launch_prefill<__half, false, HD, kPaged>(m, p, s);
}

int dispatch_prefill_e4m3_pages(int dtype, const PrefillMaps& m, const PrefillParams& p, cudaStream_t s) {
  if (p.softcap > 0.f)
    return dtype == TB200_BF16 ? launch_prefill<__nv_bfloat16, true, 128, true, true>(m, p, s)
                               : launch_prefill<__half, true, 128, true, true>(m, p, s);
  return dtype == TB200_BF16 ? launch_prefill<__nv_bfloat16, false, 128, true, true>(m, p, s)
                             : launch_prefill<__half, false, 128, true, true>(m, p, s);
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" size_t tb200_gqa_prefill_workspace_bytes(int batch, int heads, int heads_kv, int seqlen_q,
                                                    int seqlen_kv, int dim) {
  (void)batch; (void)heads; (void)heads_kv; (void)seqlen_q; (void)seqlen_kv; (void)dim;
  return 256 + 8192;  // status word (0 = ok; otherwise the code of the wait that ran out) + tuning timeline
}

extern "C" int tb200_gqa_prefill(const void* q, const void* k, const void* v, void* o, float* lse, int dtype,
                                 int batch, int seqlen_q, int seqlen_kv, int heads, int heads_kv, int dim,
                                 int is_causal, float sm_scale, float softcap, int window_left, int window_right,
                                 int flags, void* workspace, size_t workspace_bytes, void* stream) {
  if (flags < 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "flags must be a combination of TB200_PREFILL_* values");
  if (window_left < -1 || window_right < -1)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "window sizes must be -1 (unlimited) or >= 0");
  if (!q || !k || !v || !o) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "q, k, v and o must be non-null");
  if (batch <= 0 || seqlen_q <= 0 || seqlen_kv <= 0 || heads <= 0 || heads_kv <= 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "batch, seqlen_q, seqlen_kv, heads and heads_kv must be positive");
  if (heads % heads_kv != 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "heads must be divisible by heads_kv");
  if (dim != 128 && dim != 64 && dim != 256)
    TB200_FAIL(TB200_ERR_UNSUPPORTED, "head dim %d (the tcgen05 prefill kernel serves 64, 128 and 256)", dim);
  if (dtype != TB200_BF16 && dtype != TB200_F16) TB200_FAIL(TB200_ERR_UNSUPPORTED, "dtype must be F16 or BF16");
  if (!(sm_scale > 0.f)) TB200_FAIL(TB200_ERR_UNSUPPORTED, "sm_scale must be positive");
  if (softcap < 0.f) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "softcap must be non-negative");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
       reinterpret_cast<uintptr_t>(o)) & 15)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "q, k, v and o must be 16-byte aligned");
  if (!workspace || workspace_bytes < 256 + 8192) TB200_FAIL(TB200_ERR_WORKSPACE, "workspace must hold 8448 bytes");

  PrefillMaps m;
  int st;
  if ((st = make_map(&m.q, q, dtype, batch, seqlen_q, heads, dim, kBM)) != TB200_OK) return st;
  if ((st = make_map(&m.k, k, dtype, batch, seqlen_kv, heads_kv, dim, kBN)) != TB200_OK) return st;
  if ((st = make_map(&m.v, v, dtype, batch, seqlen_kv, heads_kv, dim, kBN)) != TB200_OK) return st;
  m.kp = m.k;
  m.vp = m.v;

  PrefillParams p{};
  p.o = o; p.lse = lse; p.status = static_cast<int*>(workspace);
  p.batch = batch; p.heads = heads; p.heads_kv = heads_kv; p.seqlen_q = seqlen_q; p.seqlen_kv = seqlen_kv;
  p.is_causal = is_causal; p.sm_scale = sm_scale; p.softcap = softcap;
  p.win_left = window_left; p.win_right = window_right;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (flags & TB200_PREFILL_TWO_TILES) {
    // head dim 128, on request: two Q tiles per CTA (gqa_prefill_pp.cu); it declines what it does not serve
    const int st2 = launch_prefill_pp(m, p, dtype, dim, false, s);
    if (st2 != kPrefillPpNotApplicable) return st2;
  }
  if (dim == 256) return dispatch_prefill<256, false>(dtype, m, p, s);
  return dim == 128 ? dispatch_prefill<128, false>(dtype, m, p, s) : dispatch_prefill<64, false>(dtype, m, p, s);
}

namespace {
// k_scale / v_scale non-null: the pages hold e4m3 (one fp32 scale per tensor, on the device)
int prefill_paged_impl(const void* q, const void* k_new, const void* v_new, void* k_pages,
                                       void* v_pages, void* o, float* lse, const int32_t* cu_seqlens_q,
                                       const int32_t* cu_seqlens_kv, const int32_t* cache_seqlens,
                                       const int32_t* block_table, int64_t block_table_stride, int dtype,
                                       int total_q, int total_kv, int batch, int max_seqlen_q, int heads,
                                       int heads_kv, int dim, int page_size,
                                       int64_t pool_tokens, int is_causal, float sm_scale, float softcap,
                                       int window_left, int window_right, int flags, void* workspace,
                                       size_t workspace_bytes, void* stream, const float* k_scale,
                                       const float* v_scale) {
  const bool e4m3_pages = k_scale != nullptr;
  if (flags < 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "flags must be a combination of TB200_PREFILL_* values");
  if (window_left < -1 || window_right < -1)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "window sizes must be -1 (unlimited) or >= 0");
  if (!q || !k_new || !v_new || !o || !cu_seqlens_q)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "q, k_new, v_new, o and cu_seqlens_q must be non-null");
  if (total_q <= 0 || total_kv <= 0 || batch <= 0 || max_seqlen_q <= 0 || heads <= 0 || heads_kv <= 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "total_q, total_kv, batch, max_seqlen_q, heads and heads_kv must be positive");
  if (heads % heads_kv != 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "heads must be divisible by heads_kv");
  if (dim != 128 && dim != 64 && dim != 256)
    TB200_FAIL(TB200_ERR_UNSUPPORTED, "head dim %d (the tcgen05 prefill kernel serves 64, 128 and 256)", dim);
  if (dtype != TB200_BF16 && dtype != TB200_F16) TB200_FAIL(TB200_ERR_UNSUPPORTED, "dtype must be F16 or BF16");
  if (!(sm_scale > 0.f)) TB200_FAIL(TB200_ERR_UNSUPPORTED, "sm_scale must be positive");
  if (softcap < 0.f) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "softcap must be non-negative");
  const bool has_cache = k_pages != nullptr || v_pages != nullptr || cache_seqlens != nullptr;
  if (has_cache && (window_left >= 0 || window_right >= 0))
    TB200_FAIL(TB200_ERR_UNSUPPORTED, "a sliding window over a paged cache is not served");
  if (has_cache && (cu_seqlens_kv != nullptr || total_kv != total_q))
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "with a cache, k_new / v_new hold exactly the rows of q (cu_seqlens_kv must be null)");
  if (!cu_seqlens_kv && total_kv != total_q)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "total_kv differs from total_q but cu_seqlens_kv is null");
  if (has_cache) {
    if (!k_pages || !v_pages || !cache_seqlens || !block_table)
      TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "k_pages, v_pages, cache_seqlens and block_table come together");
    if (page_size < 16 || (page_size & (page_size - 1)) != 0)
      TB200_FAIL(TB200_ERR_UNSUPPORTED, "page_size %d (a power of two >= 16 is served)", page_size);
    if (pool_tokens <= 0 || pool_tokens % page_size != 0)
      TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "pool_tokens must be a positive multiple of page_size");
    if (block_table_stride <= 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "block_table_stride must be positive");
  }
  uintptr_t bits = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_new) |
                   reinterpret_cast<uintptr_t>(v_new) | reinterpret_cast<uintptr_t>(o) |
                   reinterpret_cast<uintptr_t>(k_pages) | reinterpret_cast<uintptr_t>(v_pages);
  if (bits & 15) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "q, k_new, v_new, k_pages, v_pages and o must be 16-byte aligned");
  if (!workspace || workspace_bytes < 256 + 8192) TB200_FAIL(TB200_ERR_WORKSPACE, "workspace must hold 8448 bytes");

  PrefillMaps m;
  int st;
  if ((st = make_map(&m.q, q, dtype, 1, total_q, heads, dim, kBM)) != TB200_OK) return st;
  if ((st = make_map(&m.k, k_new, dtype, 1, total_kv, heads_kv, dim, kBN)) != TB200_OK) return st;
  if ((st = make_map(&m.v, v_new, dtype, 1, total_kv, heads_kv, dim, kBN)) != TB200_OK) return st;
  m.kp = m.k;
  m.vp = m.v;
  PrefillParams p{};
  if (has_cache) {
    p.page_box = page_size < kBN ? page_size : kBN;
    if (e4m3_pages) {
      if ((st = make_map_e4m3(&m.kp, k_pages, pool_tokens, heads_kv, dim, p.page_box)) != TB200_OK) return st;
      if ((st = make_map_e4m3(&m.vp, v_pages, pool_tokens, heads_kv, dim, p.page_box)) != TB200_OK) return st;
    } else {
      if ((st = make_map(&m.kp, k_pages, dtype, 1, pool_tokens, heads_kv, dim, p.page_box)) != TB200_OK) return st;
      if ((st = make_map(&m.vp, v_pages, dtype, 1, pool_tokens, heads_kv, dim, p.page_box)) != TB200_OK) return st;
    }
    p.page_size = page_size;
    p.page_shift = 0;
    while ((1 << p.page_shift) < page_size) ++p.page_shift;
  }
  p.o = o; p.lse = lse; p.status = static_cast<int*>(workspace);
  p.batch = batch; p.heads = heads; p.heads_kv = heads_kv; p.seqlen_q = max_seqlen_q; p.seqlen_kv = 0;
  p.is_causal = is_causal; p.sm_scale = sm_scale; p.softcap = softcap;
  p.win_left = window_left; p.win_right = window_right;
  p.cu_q = cu_seqlens_q; p.cu_kv = cu_seqlens_kv; p.cache_lens = cache_seqlens; p.bt = block_table; p.bt_stride = block_table_stride;
  p.k_new = k_new; p.v_new = v_new; p.k_pages = k_pages; p.v_pages = v_pages; p.total_q = total_q;
  p.k_scale = k_scale; p.v_scale = v_scale;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (e4m3_pages) return dispatch_prefill_e4m3_pages(dtype, m, p, s);
  if (dim == 256) return dispatch_prefill<256, true>(dtype, m, p, s);
  return dim == 128 ? dispatch_prefill<128, true>(dtype, m, p, s) : dispatch_prefill<64, true>(dtype, m, p, s);
}
}  // namespace

extern "C" int tb200_gqa_prefill_paged(const void* q, const void* k_new, const void* v_new, void* k_pages,
                                       void* v_pages, void* o, float* lse, const int32_t* cu_seqlens_q,
                                       const int32_t* cu_seqlens_kv, const int32_t* cache_seqlens,
                                       const int32_t* block_table, int64_t block_table_stride, int dtype,
                                       int total_q, int total_kv, int batch, int max_seqlen_q, int heads,
                                       int heads_kv, int dim, int page_size,
                                       int64_t pool_tokens, int is_causal, float sm_scale, float softcap,
                                       int window_left, int window_right, int flags, void* workspace,
                                       size_t workspace_bytes, void* stream) {
  return prefill_paged_impl(q, k_new, v_new, k_pages, v_pages, o, lse, cu_seqlens_q, cu_seqlens_kv, cache_seqlens,
                            block_table, block_table_stride, dtype, total_q, total_kv, batch, max_seqlen_q, heads,
                            heads_kv, dim, page_size, pool_tokens, is_causal, sm_scale, softcap, window_left,
                            window_right, flags, workspace, workspace_bytes, stream, nullptr, nullptr);
}

extern "C" int tb200_gqa_prefill_paged_e4m3_cache(const void* q, const void* k_new, const void* v_new, void* k_pages,
                                                  void* v_pages, const float* k_scale, const float* v_scale, void* o,
                                                  float* lse, const int32_t* cu_seqlens_q,
                                                  const int32_t* cache_seqlens, const int32_t* block_table,
                                                  int64_t block_table_stride, int dtype, int total_q, int batch,
                                                  int max_seqlen_q, int heads, int heads_kv, int dim, int page_size,
                                                  int64_t pool_tokens, int is_causal, float sm_scale, float softcap,
                                                  void* workspace, size_t workspace_bytes, void* stream) {
  if (!k_scale || !v_scale) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "k_scale and v_scale must be non-null (device pointers)");
  if (!k_pages || !v_pages || !cache_seqlens || !block_table)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "k_pages, v_pages, cache_seqlens and block_table must be non-null");
  if (dim != 128) TB200_FAIL(TB200_ERR_UNSUPPORTED, "head dim %d (the fused e4m3-page prefill serves 128)", dim);
  return prefill_paged_impl(q, k_new, v_new, k_pages, v_pages, o, lse, cu_seqlens_q, nullptr, cache_seqlens,
                            block_table, block_table_stride, dtype, total_q, total_q, batch, max_seqlen_q, heads,
                            heads_kv, dim, page_size, pool_tokens, is_causal, sm_scale, softcap, -1, -1, 0, workspace,
                            workspace_bytes, stream, k_scale, v_scale);
}
