// Dense GQA prefill, head dim 128, sm_100a: two 128-row Q tiles per CTA in ping-pong on one tensor
// pipe, 128-key tiles, single-pass softmax in registers, persistent grid.
//
// Role in the reference: the same as gqa_prefill.cu (GQAPrefillFwdKernel,
// src/tileops/kernels/attention/gqa_fwd.py:309-468,519-597 in tile-ai/TileOPs); the structure answers the
// reference's persistent Hopper kernel with paired M tiles (gqa_fwd_ws.py:503-1030, tile pairing at
// :634-642), rebuilt on tcgen05 / TMEM.
//
// One CTA per SM, 10 warps:
//   warps 0-3  softmax of Q tile A (thread r owns row r = TMEM lane r)
//   warps 4-7  softmax of Q tile B (the next 128 rows of the same batch element and q head)
//   warp  8    MMA issuer (one lane) and TMEM allocator
//   warp  9    TMA producer (one lane): both Q tiles once per work item, K_j / V_j into 2-stage rings
// TMEM (all 512 columns): S_A [0,128) | S_B [128,256) | O_A [256,384) | O_B [384,512).  P (16-bit, 64
// columns) overwrites the first half of its S.  The MMA lane issues, per 128-key tile j,
//     PV_A(j), QK_A(j+1), PV_B(j), QK_B(j+1)
// each pair as soon as that tile's P is ready: while the softmax warps of A work on S_A(j+1), the tensor
// pipe runs B's pair, and vice versa.  One issuer orders all MMAs, and every K/V tile in shared memory
// feeds both Q tiles.  A thread reads its whole 128-key score row from TMEM once (128 registers), takes
// the row maximum, exponentiates in place and writes P back; O is rescaled only when a row maximum grew
// by more than 2^8 (the final 1/l and the LSE use the same stale maximum, so the result is unchanged).
// S_A(j+1) is committed after PV_A(j) in issue order, so a softmax warp that sees its S also knows that
// the previous PV into its O has finished: the rescale needs no barrier of its own.
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

#ifndef TB200_PP_POLY
#define TB200_PP_POLY 0      // of every 4 exponentials on unmasked tiles, this many run on the FMA pipe
#endif

constexpr int kPM = 128;               // rows per Q tile
constexpr int kPN = 128;               // keys per KV tile
constexpr int kPD = 128;               // head dim
constexpr int kPThreads = 320;
constexpr int kPanel = 128 * 128;      // 128 rows x 128 B (64 head dims), swizzled
constexpr int kTileBytes = 2 * kPanel; // 128 x 128 16-bit
constexpr int kKvStages = 2;
struct PPSmem {
  static constexpr int q = 0;                                  // tile t, panel pn at (t * 2 + pn) * kPanel
  static constexpr int k = q + 2 * kTileBytes;
  static constexpr int v = k + kKvStages * kTileBytes;
  static constexpr int bars = v + kKvStages * kTileBytes;
  static constexpr int total = bars + 256;
};
enum { PB_QFULL = 0, PB_QEMPTY = 1, PB_KFULL = 2, PB_KEMPTY = 4, PB_VFULL = 6, PB_VEMPTY = 8, PB_SFULL = 10,
       PB_PREADY = 12, PB_OFINAL = 14, PB_COUNT = 16 };
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

// 10 warps x 192 registers fit the register file of an SM (registers are granted per warp in blocks of 512, so
// 200 would not launch; a launch bound of 320 threads would be
// rounded up to 384 and cap the kernel at 168, which spills the 128-register score row).
template <typename T, bool kSoftcap>
__global__ void __maxnreg__(192)
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
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(PB_KFULL + s), 1);
      mbar_init(bar(PB_KEMPTY + s), 1);
      mbar_init(bar(PB_VFULL + s), 1);
      mbar_init(bar(PB_VEMPTY + s), 1);
      mbar_init(bar(PB_SFULL + s), 1);
      mbar_init(bar(PB_PREADY + s), 128);
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
  constexpr uint32_t idesc_pv = make_idesc(fmt, 1, kPD);

  if (warp == 9) {
    // ================= TMA producer =================
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      uint32_t nq = 0, kc = 0, vc = 0;
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
        auto load_tile = [&](uint32_t dst, const CUtensorMap* map, uint32_t full_bar, int j) {
#pragma unroll
          for (int pn = 0; pn < 2; ++pn)
#pragma unroll
            for (int r = 0; r < 2; ++r)
              tma_load_4d(dst + pn * kPanel + r * 64 * 128, map, full_bar, pn * 64, it.hk, j * kPN + r * 64, it.b);
        };
        for (int j = it.jlo; j < it.jhi; ++j) {
          const int ks = kc & 1, vs = vc & 1;
          if (!wait(PB_KEMPTY + ks, ((kc >> 1) & 1) ^ 1, 702)) { ok = false; break; }
          mbar_expect_tx(bar(PB_KFULL + ks), kTileBytes);
          load_tile(sbase + PPSmem::k + ks * kTileBytes, &map_k, bar(PB_KFULL + ks), j);
          ++kc;
          if (!wait(PB_VEMPTY + vs, ((vc >> 1) & 1) ^ 1, 703)) { ok = false; break; }
          mbar_expect_tx(bar(PB_VFULL + vs), kTileBytes);
          load_tile(sbase + PPSmem::v + vs * kTileBytes, &map_v, bar(PB_VFULL + vs), j);
          ++vc;
        }
      }
    }
  } else if (warp == 8) {
    // ================= MMA issuer =================
    if (lane == 0) {
      uint32_t nq = 0, kc = 0, vc = 0, pc[2] = {0, 0};
      const uint64_t dq0 = make_desc(sbase + PPSmem::q, 16, 1024);
      const uint64_t dk0 = make_desc(sbase + PPSmem::k, 16, 1024);
      const uint64_t dv0 = make_desc(sbase + PPSmem::v, kPanel, 1024);
      constexpr uint64_t kTileStep = kTileBytes >> 4;      // next tile / stage, in start-address units
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_items; item += gridDim.x) {
        const PPItem it = pp_item(p, item);
        if (it.jhi <= it.jlo) continue;
        // S_t = Q_t K^T from K stage ks
        auto issue_qk = [&](int t, int ks) {
#pragma unroll
          for (int kk = 0; kk < kPD / 16; ++kk) {
            // K-major operands: 16 elements per step = 32 B inside the 128 B swizzled row; after 4
            // steps the second 64-element panel (16 KB further)
            const uint32_t o = ((kk >> 2) * kPanel + (kk & 3) * 32) >> 4;
            tc_mma_ss(tmem + kColSA + t * kPN, dq0 + t * kTileStep + o, dk0 + ks * kTileStep + o, idesc_qk, kk > 0 ? 1u : 0u);
          }
          tc_commit(bar(PB_SFULL + t));
        };
        if (!wait(PB_QFULL, nq & 1, 711)) break;
        ++nq;
        {
          // first key tile of the item
          const int ks = kc & 1;
          if (!wait(PB_KFULL + ks, (kc >> 1) & 1, 712)) break;
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < 2; ++t)
            if (it.jlo >= it.lo[t] && it.jlo < it.hi[t]) issue_qk(t, ks);
          tc_commit(bar(PB_KEMPTY + ks));
          ++kc;
          if (it.jlo + 1 == it.jhi) tc_commit(bar(PB_QEMPTY));
        }
        for (int j = it.jlo; ok && j < it.jhi; ++j) {
          const int vs = vc & 1, ks = kc & 1;
          const bool more = j + 1 < it.jhi;
          if (!wait(PB_VFULL + vs, (vc >> 1) & 1, 713)) { ok = false; break; }
          if (more && !wait(PB_KFULL + ks, (kc >> 1) & 1, 714)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j >= it.lo[t] && j < it.hi[t]) {
              if (!wait(PB_PREADY + t, pc[t] & 1, 715)) { ok = false; break; }
              ++pc[t];
              tc_fence_after();
#pragma unroll
              for (int kk = 0; kk < kPN / 16; ++kk) {
                // B = V: MN-major, 16 keys per step = 16 rows of 128 B; the two 64-wide d panels are
                // kPanel apart (leading offset), 8-row groups 1024 B apart (stride offset)
                tc_mma_ts(tmem + kColOA + t * kPD, tmem + kColSA + t * kPN + kk * 8,
                          dv0 + vs * kTileStep + ((kk * 2048) >> 4), idesc_pv, (j > it.lo[t] || kk > 0) ? 1u : 0u);
              }
              if (j == it.hi[t] - 1) tc_commit(bar(PB_OFINAL + t));
            }
            if (more && j + 1 >= it.lo[t] && j + 1 < it.hi[t]) issue_qk(t, ks);
          }
          if (!ok) break;
          tc_commit(bar(PB_VEMPTY + vs));
          ++vc;
          if (more) {
            tc_commit(bar(PB_KEMPTY + ks));
            ++kc;
            if (j + 2 == it.jhi) tc_commit(bar(PB_QEMPTY));   // the last QKs of the item are issued
          }
        }
      }
    }
  } else {
    // ================= softmax / rescale / epilogue (thread = row of tile t) =================
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
    uint32_t cs = 0, co = 0;
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
        const int k0 = j * kPN;
        const bool need_mask = (has_upper && k0 + kPN - 1 > m0 + off + up_extra) || (k0 + kPN > p.seqlen_kv) ||
                               (p.win_left >= 0 && k0 < m0 + kPM - 1 + off - p.win_left);
        uint32_t s[4][32];
#pragma unroll
        for (int cg = 0; cg < 4; ++cg) tc_ld32(s_addr + cg * 32, s[cg]);
#pragma unroll
        for (int cg = 0; cg < 4; ++cg) tc_wait_ld(s[cg]);
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
        if (__any_sync(0xffffffffu, grow)) {
          // 1 for a row that still has seen no key (avoids inf - inf), 0 for a row seeing its first
          const float alpha = (m_new == -INFINITY) ? 1.f : fast_exp2((m_run - m_new) * c);
          l_run *= alpha;
          if (j > it.lo[t]) {
            // PV(j-1) has finished: S(j) was committed behind it
#pragma unroll
            for (int cg = 0; cg < kPD / 32; ++cg) {
              uint32_t ov[32];
              tc_ld32(o_addr + cg * 32, ov);
              tc_wait_ld(ov);
#pragma unroll
              for (int e = 0; e < 32; ++e) ov[e] = __float_as_uint(__uint_as_float(ov[e]) * alpha);
              tc_st32(o_addr + cg * 32, ov);
            }
          }
          m_run = m_new;
        }
        const float neg_mc = (m_run == -INFINITY) ? 0.f : -m_run * c;

        // ---- p = 2^(s*c - m*c), row sum, P (16-bit) over the first 64 columns of S ----
        uint64_t lsum_a = 0, lsum_b = 0;                    // two (even key, odd key) pairs of partial sums
        const uint64_t c2 = f2_pack(c, c), neg_mc2 = f2_pack(neg_mc, neg_mc);
        const bool poly_ok = TB200_PP_POLY > 0 && !need_mask;   // the polynomial needs finite inputs
#pragma unroll
        for (int cg = 0; cg < 4; ++cg) {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            float x0, x1;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(s[cg][2 * e]), __uint_as_float(s[cg][2 * e + 1])), c2, neg_mc2), x0, x1);
            float p0, p1;
            if (TB200_PP_POLY > 0 && (e & 1) == 1 && poly_ok) {
              p0 = (TB200_PP_POLY >= 2) ? exp2_poly(x0) : fast_exp2(x0);
              p1 = exp2_poly(x1);
            } else {
              p0 = fast_exp2(x0);
              p1 = fast_exp2(x1);
            }
            if (e & 1) lsum_b = f2_add(lsum_b, f2_pack(p0, p1)); else lsum_a = f2_add(lsum_a, f2_pack(p0, p1));
            pk[e] = pack2<T>(p0, p1);
          }
          tc_st16(s_addr + cg * 16, pk);
        }
        float lsum0, lsum1;
        f2_unpack(f2_add(lsum_a, lsum_b), lsum0, lsum1);
        l_run += lsum0 + lsum1;
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar(PB_PREADY + t));
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
