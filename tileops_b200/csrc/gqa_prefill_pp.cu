// Dense GQA prefill, head dim 128, sm_100a: two 128-row Q tiles per CTA on one tensor pipe, 128-key tiles,
// single-pass softmax in registers, P handed to the second product through shared memory, persistent grid.
//
// Role in the reference: the same as gqa_prefill.cu (GQAPrefillFwdKernel,
// src/tileops/kernels/attention/gqa_fwd.py:309-468,519-597 in tile-ai/TileOPs); the structure answers the
// reference's persistent Hopper kernel with paired M tiles (gqa_fwd_ws.py:503-1030, tile pairing at
// :634-642), rebuilt on tcgen05 / TMEM.
//
// What shapes the design: on B200 a tcgen05.mma with M = 128, K = 16 occupies the tensor pipe for at least
// ~96 clocks whatever N is (N = 64: 96, N = 128: 96-107, N = 256: 138-171; tb200_mma_issue_probe measures
// it), so the number of MMA instructions per key, not their size, bounds the kernel.  The kernel of
// gqa_prefill.cu (64-key tiles, N = 64 score products) issues 12 per 64 keys and runs at that bound;
// 128-key tiles need 16 per 128 keys.  With 128-key tiles TMEM holds S and O of two Q tiles exactly once
// (4 x 128 columns), so S cannot be double buffered; instead S is released early:
//
// One CTA per SM, 12 warps (the last two only complete the third warpgroup):
//   warps 0-3  softmax of Q tile A (thread r owns row r = TMEM lane r)
//   warps 4-7  softmax of Q tile B (the next 128 rows of the same batch element and q head)
//   warp  8    MMA issuer (one lane) and TMEM allocator
//   warp  9    TMA producer (one lane): both Q tiles once per work item, K / V tiles into one 3-slot ring
// TMEM (all 512 columns): S_A [0,128) | S_B [128,256) | O_A [256,384) | O_B [384,512).
// A softmax thread reads its whole 128-key score row from TMEM once (128 registers) and at once arrives on
// S_FREE: the MMA lane may then overwrite S with the NEXT tile's scores while this tile's row maximum,
// exponentials and row sum are computed from registers.  P (16-bit) goes to a swizzled shared-memory tile
// (the K-major A operand of O += P V), so the second product does not touch S either.  Per 128-key tile j
// the MMA lane issues QK_A(j+1), QK_B(j+1), PV_A(j), PV_B(j): the score products run under the softmax of
// the tile before, the PV products under the softmax of the tile after, and a softmax warp that finishes a
// tile finds its next S ready.  O is rescaled only when a row maximum grew by more than 2^8 (the final 1/l
// and the LSE use the same stale maximum, so the result is unchanged); the rescale waits for the previous
// PV through the PV_DONE barrier, which also guards the reuse of the P tile.
//
// The grid is persistent (one CTA per SM); CTA c takes work items c, c + grid, ... of a list sorted
// heaviest first (last row pairs first).  The TMA and MMA lanes run ahead into the next item (its Q and
// first K tile are loaded and QK(0) issued while the softmax warps write the current item's output), so
// consecutive items overlap without a second resident CTA.
//
// Every mbarrier wait is bounded; on a timeout the CTA records a code (7xx) in the status word, the
// roles leave their loops, copies in flight get time to land, TMEM is freed and the CTA returns.
#include <type_traits>

#include "gqa_prefill.cuh"

namespace tb200 {
namespace {

// Optional timeline for tuning (-DTB200_TRACE): CTA 0 stamps clock64() at the milestones of its MMA lane
// (slots 10-13: score product and PV product issued, per tile) and of the first thread of each softmax
// warpgroup (slots 0-4 and 5-9: S seen, S read, maximum done, exponentials done, P handed over) for the first
// kTraceIters key tiles of its first work item into the workspace behind the status word.
#ifdef TB200_TRACE
constexpr int kTraceIters = 40, kTraceSlots = 14;
#define TB200_PP_STAMP(slot, j)                                                                       \
  do {                                                                                                \
    if (blockIdx.x == 0 && item == int(blockIdx.x) && (j) < kTraceIters)                              \
      reinterpret_cast<long long*>(p.status + 64)[(j) * kTraceSlots + (slot)] = clock64();            \
  } while (0)
#else
#define TB200_PP_STAMP(slot, j) do {} while (0)
#endif

constexpr int kPM = 128;               // rows per Q tile
constexpr int kPN = 128;               // keys per KV tile
constexpr int kPD = 128;               // head dim
constexpr int kPThreads = 384;
constexpr int kLaunchRegs = 168;       // what ptxas grants 384 threads per CTA
constexpr int kSoftmaxRegs = 224;      // softmax warpgroups after setmaxnreg.inc
constexpr int kIssueRegs = 56;         // MMA / TMA warpgroup after setmaxnreg.dec
static_assert(2 * kSoftmaxRegs + kIssueRegs <= 3 * kLaunchRegs, "setmaxnreg.inc would block forever");
static_assert(kSoftmaxRegs % 8 == 0 && kIssueRegs % 8 == 0 && kIssueRegs >= 24 && kSoftmaxRegs <= 256, "setmaxnreg operand");
constexpr int kPanel = 128 * 128;      // 128 rows x 128 B (64 head dims or 64 keys), swizzled
constexpr int kTileBytes = 2 * kPanel; // 128 x 128 16-bit
constexpr int kRing = 3;               // K / V tiles in flight: K_j+1, V_j and the next one
struct PPSmem {
  static constexpr int q = 0;                                  // tile t, panel pn at (t * 2 + pn) * kPanel
  static constexpr int ring = q + 2 * kTileBytes;              // K_lo, K_lo+1, V_lo, K_lo+2, V_lo+1, ... round robin
  static constexpr int pt = ring + kRing * kTileBytes;         // P of tile t (K-major: rows x 128 keys)
  static constexpr int bars = pt + 2 * kTileBytes;
  static constexpr int total = bars + 256;
};
enum { PB_QFULL = 0, PB_QEMPTY = 1, PB_RFULL = 2, PB_REMPTY = 5, PB_SFULL = 8, PB_SFREE = 10, PB_PREADY = 12,
       PB_PVDONE = 14, PB_OFINAL = 16, PB_COUNT = 18 };
constexpr uint32_t kColSA = 0, kColOA = 256;   // tile t: S at 128 t, O at 256 + 128 t

// One work item: a pair of Q tiles of one (batch element, q head), and the key tiles each of them sees.
struct PPItem {
  int b, h, hk;
  int m0[2];          // first row of the tile
  int lo[2], hi[2];   // key tiles [lo, hi) the tile sees; hi <= lo: none (rows masked out entirely, or no rows)
  int jlo, jhi;       // union over both tiles
};
__device__ __forceinline__ PPItem pp_item(const PrefillParams& p, int item) {
  PPItem it;
  const int n_pairs = (p.seqlen_q + 2 * kPM - 1) / (2 * kPM);
  const int per = p.heads * p.batch;
  const int pair = n_pairs - 1 - item / per;          // heaviest (last) row pairs first
  const int rest = item % per;
  it.b = rest / p.heads;
  it.h = rest % p.heads;
  it.hk = it.h / (p.heads / p.heads_kv);
  const int off = p.seqlen_kv - p.seqlen_q;           // bottom-right alignment
  const bool has_upper = p.is_causal || p.win_right >= 0;
  const int up_extra = p.is_causal ? 0 : p.win_right;
  const int n_all = (p.seqlen_kv + kPN - 1) / kPN;
  it.jlo = 0x7fffffff; it.jhi = 0;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int m0 = pair * 2 * kPM + t * kPM;
    it.m0[t] = m0;
    int hi = n_all, lo = 0;
    if (has_upper) {
      const long long last_key = (long long)m0 + kPM - 1 + off + up_extra;   // of the tile's last row
      hi = last_key < 0 ? 0 : int(min((long long)hi, last_key / kPN + 1));
    }
    if (p.win_left >= 0) lo = max(0, m0 + off - p.win_left) / kPN;
    if (m0 >= p.seqlen_q) { lo = 0; hi = 0; }
    it.lo[t] = lo; it.hi[t] = hi;
    if (hi > lo) { it.jlo = min(it.jlo, lo); it.jhi = max(it.jhi, hi); }
  }
  if (it.jhi == 0) it.jlo = 0;
  return it;
}

// Registers: each of the four SM sub-partitions holds 16384 and hosts a quarter of the warps, so 12 warps
// launch with 168 registers each.  The third warpgroup (MMA lane, TMA lane, two idle warps) then gives
// registers back (setmaxnreg.dec) and the two softmax warpgroups take them (setmaxnreg.inc), which makes
// room for the 128-register score row.  setmaxnreg.inc BLOCKS until the CTA's own pool - what it was
// launched with, 3 x 168 per lane, not the SM's register file - has the registers, so the new counts must
// add up to at most that (checked below), or the kernel would wait forever.
template <typename T, bool kSoftcap>
__global__ void __launch_bounds__(kPThreads, 1)
gqa_prefill_pp_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, PrefillParams p, int total_items) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t sbase = smem_u32(smem);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + PPSmem::bars);
  uint32_t* s_tmem = reinterpret_cast<uint32_t*>(bars + PB_COUNT);
  volatile int* s_abort = reinterpret_cast<volatile int*>(s_tmem + 1);
  auto bar = [&](int i) { return smem_u32(bars + i); };
  auto wait = [&](int b, uint32_t parity, int code) {
    return mbar_wait_bounded(bar(b), parity, s_abort, p.status, code, kWaitCycles);
  };

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  __shared__ int s_skip;
  if (tid == 0) s_skip = *reinterpret_cast<volatile int*>(p.status);
  __syncthreads();
  if (s_skip != 0) return;   // an earlier launch gave up on a wait: do not start more work

  if (tid == 0) {
    mbar_init(bar(PB_QFULL), 1);
    mbar_init(bar(PB_QEMPTY), 1);
    for (int s = 0; s < kRing; ++s) {
      mbar_init(bar(PB_RFULL + s), 1);
      mbar_init(bar(PB_REMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(PB_SFULL + s), 1);
      mbar_init(bar(PB_SFREE + s), 128);
      mbar_init(bar(PB_PREADY + s), 128);
      mbar_init(bar(PB_PVDONE + s), 1);
      mbar_init(bar(PB_OFINAL + s), 1);
    }
    *s_abort = 0;
    mbar_fence_init();
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(s_tmem)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *s_tmem;

  constexpr uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
  constexpr uint32_t idesc_qk = make_idesc(fmt, 0, kPN);
  // (An MMA whose A and B element formats differ - f16 P against bf16 V - is an illegal instruction on
  // sm_100a: P always has the type of V.)
  constexpr bool kHalfP = std::is_same<T, __half>::value;
  constexpr uint32_t idesc_pv = make_idesc(fmt, 1, kPD);

  if (warp >= 8) {
    // third warpgroup: TMA lane, MMA lane and two idle warps (a register hand-over needs whole warpgroups)
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kIssueRegs));
   if (warp == 9) {
    // ================= TMA producer =================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      uint32_t nq = 0, rc = 0;                     // work items and ring tiles loaded so far
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const PPItem it = pp_item(p, item);
        if (it.jhi <= it.jlo) continue;
        if (!wait(PB_QEMPTY, (nq & 1) ^ 1, 701)) break;
        mbar_expect_tx(bar(PB_QFULL), 2 * kTileBytes);
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
          for (int pn = 0; pn < 2; ++pn)
            tma_load_4d(sbase + PPSmem::q + (t * 2 + pn) * kPanel, &map_q, bar(PB_QFULL), pn * 64, it.h, it.m0[t], it.b);
        ++nq;
        // a 128-key tile is two 64-row boxes per 64-dim panel (the maps describe 64-row boxes)
        auto load_tile = [&](const CUtensorMap* map, int j) -> bool {
          const int slot = rc % kRing;
          if (!wait(PB_REMPTY + slot, ((rc / kRing) & 1) ^ 1, 702)) return false;
          mbar_expect_tx(bar(PB_RFULL + slot), kTileBytes);
          const uint32_t dst = sbase + PPSmem::ring + slot * kTileBytes;
#pragma unroll
          for (int pn = 0; pn < 2; ++pn)
#pragma unroll
            for (int r = 0; r < 2; ++r)
              tma_load_4d(dst + pn * kPanel + r * 64 * 128, map, bar(PB_RFULL + slot), pn * 64, it.hk, j * kPN + r * 64, it.b);
          ++rc;
          return true;
        };
        // the order the MMA lane consumes them in: K_lo, then K_j+1 and V_j for every tile j
        if (!load_tile(&map_k, it.jlo)) break;
        for (int j = it.jlo; j < it.jhi; ++j) {
          if (j + 1 < it.jhi && !load_tile(&map_k, j + 1)) { ok = false; break; }
          if (!load_tile(&map_v, j)) { ok = false; break; }
        }
      }
    }
  } else if (warp == 8) {
    // ================= MMA issuer =================
    if (lane == 0) {
      uint32_t nq = 0, rc = 0;                     // work items and ring tiles consumed so far
      uint32_t qk_n[2] = {0, 0}, pv_n[2] = {0, 0}; // score products and PV products issued so far, per Q tile
      const uint64_t dq0 = make_desc(sbase + PPSmem::q, 16, 1024);
      const uint64_t dp0 = make_desc(sbase + PPSmem::pt, 16, 1024);
      constexpr uint64_t kTileStep = kTileBytes >> 4;      // next tile / slot, in start-address units
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const PPItem it = pp_item(p, item);
        if (it.jhi <= it.jlo) continue;
        // S_t(j) = Q_t K_j^T for the tiles that see key tile j; K_j is the ring's next tile
        auto issue_qk = [&](int j) -> bool {
          const int slot = rc % kRing;
          if (!wait(PB_RFULL + slot, (rc / kRing) & 1, 712)) return false;
          const uint64_t dk = make_desc(sbase + PPSmem::ring + slot * kTileBytes, 16, 1024);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j < it.lo[t] || j >= it.hi[t]) continue;
            // the softmax warps must have read the previous scores of this tile out of TMEM
            if (qk_n[t] > 0 && !wait(PB_SFREE + t, (qk_n[t] - 1) & 1, 713)) return false;
            ++qk_n[t];
            tc_fence_after();
            // K-major operands: 16 elements per step = 32 B inside the 128 B swizzled row; after 4 steps the
            // second 64-element panel (16 KB further)
            tc_mma_ss_x8<(kPanel >> 4), (kPanel >> 4)>(tmem + kColSA + t * kPN, dq0 + t * kTileStep, dk, idesc_qk);
            tc_commit(bar(PB_SFULL + t));
            TB200_PP_STAMP(10 + 2 * t, j - it.jlo);
          }
          tc_commit(bar(PB_REMPTY + slot));
          ++rc;
          if (j + 1 == it.jhi) tc_commit(bar(PB_QEMPTY));     // the last score products of the item are issued
          return true;
        };
        if (!wait(PB_QFULL, nq & 1, 711)) break;
        ++nq;
        if (!issue_qk(it.jlo)) break;
        for (int j = it.jlo; ok && j < it.jhi; ++j) {
          if (j + 1 < it.jhi && !issue_qk(j + 1)) { ok = false; break; }
          // O_t += P_t(j) V_j; V_j is the ring's next tile
          const int slot = rc % kRing;
          if (!wait(PB_RFULL + slot, (rc / kRing) & 1, 714)) { ok = false; break; }
          const uint64_t dv = make_desc(sbase + PPSmem::ring + slot * kTileBytes, kPanel, 1024);
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j < it.lo[t] || j >= it.hi[t]) continue;
            if (!wait(PB_PREADY + t, pv_n[t] & 1, 715)) { ok = false; break; }
            ++pv_n[t];
            tc_fence_after();
            // A = P (K-major, like Q); B = V: MN-major, 16 keys per step = 16 rows of 128 B; the two 64-wide d
            // panels are kPanel apart (leading offset), 8-row groups 1024 B apart (stride offset)
            tc_mma_ss_pv_x8<(kPanel >> 4), (2048 >> 4)>(tmem + kColOA + t * kPD, dp0 + t * kTileStep, dv, idesc_pv,
                                                        j > it.lo[t] ? 1u : 0u);
            tc_commit(bar(PB_PVDONE + t));
            if (j == it.hi[t] - 1) tc_commit(bar(PB_OFINAL + t));
            TB200_PP_STAMP(11 + 2 * t, j - it.jlo);
          }
          if (!ok) break;
          tc_commit(bar(PB_REMPTY + slot));
          ++rc;
        }
      }
    }
   }
  } else {
    // ================= softmax / rescale / epilogue (thread = row of tile t) =================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int t = warp >> 2;                                // 0: tile A, 1: tile B
    const int row = tid & 127;                              // == TMEM lane
    const uint32_t lane_addr = uint32_t((warp & 3) * 32) << 16;
    const uint32_t s_addr = tmem + lane_addr + kColSA + t * kPN;
    const uint32_t o_addr = tmem + lane_addr + kColOA + t * kPD;
    const float cap = p.softcap;
    const float c = kSoftcap ? kLog2e : p.sm_scale * kLog2e;   // multiplies the raw (or capped) score
    const float pre = kSoftcap ? p.sm_scale / cap : 0.f;
    const int off = p.seqlen_kv - p.seqlen_q;
    const bool has_upper = p.is_causal || p.win_right >= 0;
    const int up_extra = p.is_causal ? 0 : p.win_right;
    uint32_t cs = 0, co = 0, pw = 0;                        // S tiles read, outputs written, P tiles written so far
    bool ok = true;

    for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
      const PPItem it = pp_item(p, item);
      const int m0 = it.m0[t];
      const int q_idx = m0 + row;
      if (m0 >= p.seqlen_q) continue;
      T* orow = reinterpret_cast<T*>(p.o) + ((size_t(it.b) * p.seqlen_q + q_idx) * p.heads + it.h) * kPD;
      float* lse_ptr = p.lse ? p.lse + (size_t(it.b) * p.heads + it.h) * p.seqlen_q + q_idx : nullptr;
      if (it.hi[t] <= it.lo[t]) {
        // every key of the whole row tile is masked: zeros, LSE = -inf
        if (q_idx < p.seqlen_q) {
          const uint4 z = make_uint4(0, 0, 0, 0);
          for (int e = 0; e < kPD; e += 8) *reinterpret_cast<uint4*>(orow + e) = z;
          if (lse_ptr) *lse_ptr = -INFINITY;
        }
        continue;
      }
      const int key_limit = has_upper ? q_idx + off + up_extra : 0x7fffffff;   // last visible key of this row
      const int key_floor = p.win_left >= 0 ? q_idx + off - p.win_left : int(0x80000000);
      float m_run = -INFINITY, l_run = 0.f;   // m_run: the maximum O and l are currently scaled to

      for (int j = it.lo[t]; j < it.hi[t]; ++j) {
        // the warp leaves the loop together: the TMEM loads below are warp-collective
        if (!__all_sync(0xffffffffu, wait(PB_SFULL + t, cs & 1, 721))) { ok = false; break; }
        ++cs;
        tc_fence_after();
        if (row == 0) TB200_PP_STAMP(5 * t + 0, j - it.jlo);
        const int k0 = j * kPN;
        const bool need_mask = (has_upper && k0 + kPN - 1 > m0 + off + up_extra) || (k0 + kPN > p.seqlen_kv) ||
                               (p.win_left >= 0 && k0 < m0 + kPM - 1 + off - p.win_left);
        uint32_t s[4][32];
#pragma unroll
        for (int cg = 0; cg < 4; ++cg) tc_ld32(s_addr + cg * 32, s[cg]);
#pragma unroll
        for (int cg = 0; cg < 4; ++cg) tc_wait_ld(s[cg]);
        // the scores are in registers: S may be overwritten with the next tile's
        tc_fence_before();
        mbar_arrive(bar(PB_SFREE + t));
        if (row == 0) TB200_PP_STAMP(5 * t + 1, j - it.jlo);
        if (kSoftcap) {
#pragma unroll
          for (int cg = 0; cg < 4; ++cg)
#pragma unroll
            for (int e = 0; e < 32; ++e) s[cg][e] = __float_as_uint(cap * fast_tanh(__uint_as_float(s[cg][e]) * pre));
        }
        if (need_mask) {
#pragma unroll
          for (int cg = 0; cg < 4; ++cg)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int key = k0 + cg * 32 + e;
              if (key > key_limit || key < key_floor || key >= p.seqlen_kv) s[cg][e] = 0xff800000u;   // -inf
            }
        }
        // ---- row maximum (four independent chains) ----
        float mx;
        {
          float a[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
          for (int cg = 0; cg < 4; ++cg)
#pragma unroll
            for (int e = 0; e < 32; e += 2) a[cg] = max3(a[cg], __uint_as_float(s[cg][e]), __uint_as_float(s[cg][e + 1]));
          mx = fmaxf(fmaxf(a[0], a[1]), fmaxf(a[2], a[3]));
        }
        // ---- does the running maximum move (and O have to be rescaled)? ----
        const float m_new = fmaxf(m_run, mx);
        const bool grow = (m_new - m_run) * c > kRescaleThreshold || (m_run == -INFINITY && m_new != -INFINITY);
        bool pv_waited = false;
        if (__any_sync(0xffffffffu, grow)) {
          // 1 for a row that still has seen no key (avoids inf - inf), 0 for a row seeing its first
          const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2((m_run - m_new) * c);
          l_run *= alpha;
          if (j > it.lo[t]) {
            // the previous PV of this tile may still be adding into O
            if (!__all_sync(0xffffffffu, wait(PB_PVDONE + t, (pw - 1) & 1, 723))) { ok = false; break; }
            pv_waited = true;
            tc_fence_after();
#pragma unroll
            for (int cg = 0; cg < kPD / 32; ++cg) {
              uint32_t ov[32];
              tc_ld32(o_addr + cg * 32, ov);
              tc_wait_ld(ov);
#pragma unroll
              for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
              tc_st32(o_addr + cg * 32, ov);
            }
            tc_wait_st();
          }
          m_run = m_new;
        }
        const float neg_mc = (m_run == -INFINITY) ? 0.f : -m_run * c;
        if (row == 0) TB200_PP_STAMP(5 * t + 2, j - it.jlo);

        // ---- p = 2^(s*c - m*c), row sum; P (16-bit) stays in registers until its shared-memory tile is free ----
        uint32_t pk[4][16];
        {
          uint64_t lsum_a = 0, lsum_b = 0;                    // two (even key, odd key) pairs of partial sums
          const uint64_t c2 = f2_pack(c, c), neg_mc2 = f2_pack(neg_mc, neg_mc);
#pragma unroll
          for (int cg = 0; cg < 4; ++cg)
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              float x0, x1;
              f2_unpack(f2_fma(f2_pack(__uint_as_float(s[cg][2 * e]), __uint_as_float(s[cg][2 * e + 1])), c2, neg_mc2), x0, x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              if (e & 1) lsum_b = f2_add(lsum_b, f2_pack(p0, p1)); else lsum_a = f2_add(lsum_a, f2_pack(p0, p1));
              pk[cg][e] = pack2<T>(p0, p1);
            }
          float lsum0, lsum1;
          f2_unpack(f2_add(lsum_a, lsum_b), lsum0, lsum1);
          l_run += lsum0 + lsum1;
        }
        if (row == 0) TB200_PP_STAMP(5 * t + 3, j - it.jlo);
        // the PV product that read the previous P of this tile must be done before the tile is rewritten
        if (pw > 0 && !pv_waited) {
          if (!__all_sync(0xffffffffu, wait(PB_PVDONE + t, (pw - 1) & 1, 724))) { ok = false; break; }
        }
        ++pw;
        {
          // row r of the K-major P tile: 128 B per 64-key panel, 16-byte chunk c at (c ^ (r & 7)) * 16
          unsigned char* prow = smem + PPSmem::pt + t * kTileBytes + row * 128;
          const int x = row & 7;
#pragma unroll
          for (int cg = 0; cg < 4; ++cg)
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const int chunk = cg * 4 + q4;                  // 8 keys per chunk, 16 chunks per row
              *reinterpret_cast<uint4*>(prow + (chunk >> 3) * kPanel + (((chunk & 7) ^ x) << 4)) =
                  make_uint4(pk[cg][q4 * 4], pk[cg][q4 * 4 + 1], pk[cg][q4 * 4 + 2], pk[cg][q4 * 4 + 3]);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic stores, read by the MMA's async proxy
        mbar_arrive(bar(PB_PREADY + t));
        if (row == 0) TB200_PP_STAMP(5 * t + 4, j - it.jlo);
      }
      if (!ok) break;

      // ---- epilogue: O / l -> global, LSE ----
      if (!__all_sync(0xffffffffu, wait(PB_OFINAL + t, co & 1, 722))) { ok = false; break; }
      ++co;
      tc_fence_after();
      const float inv_l = l_run > 0.f ? 1.f / l_run : 0.f;
#pragma unroll
      for (int cg = 0; cg < kPD / 32; ++cg) {
        uint32_t ov[32];
        tc_ld32(o_addr + cg * 32, ov);
        tc_wait_ld(ov);
        if (q_idx < p.seqlen_q) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(ov[e]) * inv_l, __uint_as_float(ov[e + 1]) * inv_l);
            w.y = pack2<T>(__uint_as_float(ov[e + 2]) * inv_l, __uint_as_float(ov[e + 3]) * inv_l);
            w.z = pack2<T>(__uint_as_float(ov[e + 4]) * inv_l, __uint_as_float(ov[e + 5]) * inv_l);
            w.w = pack2<T>(__uint_as_float(ov[e + 6]) * inv_l, __uint_as_float(ov[e + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + cg * 32 + e) = w;
          }
        }
      }
      if (lse_ptr && q_idx < p.seqlen_q) *lse_ptr = l_run > 0.f ? m_run * c + log2f(l_run) : -INFINITY;
      // the O reads above are complete (wait::ld) before this warp's next arrival on P_READY lets the
      // next item's first PV overwrite O
      tc_fence_before();
    }
  }

  // ---- teardown -----------------------------------------------------------------------
  __syncwarp();   // the single-lane roles rejoin their warps before the block-wide barrier
  tc_fence_before();
  __syncthreads();
  if (*s_abort) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);   // copies still in flight land before the shared memory goes
  }
  if (warp == 8) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
}

template <typename T, bool kSoftcap>
int launch_pp(const PrefillMaps& m, const PrefillParams& p, cudaStream_t stream) {
  auto kern = gqa_prefill_pp_kernel<T, kSoftcap>;
  const int smem = PPSmem::total + 1024;
  static thread_local bool configured[64] = {false};
  int dev = 0;
  TB200_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return kPrefillPpNotApplicable;
  if (!configured[dev]) {
    TB200_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured[dev] = true;
  }
  const long long n_pairs = (p.seqlen_q + 2 * kPM - 1) / (2 * kPM);
  const long long total = n_pairs * p.heads * p.batch;
  if (total > 0x7fffffffLL) return kPrefillPpNotApplicable;
  const int grid = int(total < sm_count() ? total : sm_count());
  kern<<<grid, kPThreads, smem, stream>>>(m.q, m.k, m.v, p, int(total));
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}

}  // namespace

int launch_prefill_pp(const PrefillMaps& m, const PrefillParams& p, int dtype, int head_dim, bool paged,
                      cudaStream_t stream) {
  if (paged || head_dim != kPD) return kPrefillPpNotApplicable;
  if (p.softcap > 0.f)
    return dtype == TB200_BF16 ? launch_pp<__nv_bfloat16, true>(m, p, stream) : launch_pp<__half, true>(m, p, stream);
  return dtype == TB200_BF16 ? launch_pp<__nv_bfloat16, false>(m, p, stream) : launch_pp<__half, false>(m, p, stream);
}

}  // namespace tb200
