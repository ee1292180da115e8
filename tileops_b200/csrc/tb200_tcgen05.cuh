// tcgen05 / TMEM wrappers (sm_100a) shared by the prefill kernels: MMA issue from shared-memory and
// TMEM operands, TMEM loads and stores, commit, fences, the shared-memory matrix descriptor and the
// instruction descriptor of kind::f16, and the packed two-wide fp32 arithmetic.
#pragma once

#include "tb200_async.cuh"

namespace tb200 {

#ifndef TB200_PF_TIE
#define TB200_PF_TIE 1
#endif

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Eight MMAs of one 128-deep contraction in a single asm block, so that the issuing lane spends three
// instructions per MMA (two address adds and the MMA) instead of a compiler-scheduled sequence per call:
// with two busy softmax warps on the same scheduler every extra instruction of the issuing lane waits for
// an issue slot, and the tensor pipe idles between MMAs.
//   tc_mma_ss_x8: D[tmem] = A[smem] B[smem] over 8 k-steps of 16 elements; both operands K-major with 128 B
//   rows: step kk sits (kk & 3) * 32 B into the row and (kk >> 2) panels further (A_PANEL / B_PANEL are the
//   panel sizes in descriptor units, bytes >> 4).  The first step overwrites D, the rest accumulate.
template <uint32_t A_PANEL, uint32_t B_PANEL>
__device__ __forceinline__ void tc_mma_ss_x8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a, b;\n\t"
      "setp.ne.b32 p0, %3, %3;\n\tsetp.eq.b32 p1, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
      "add.s64 a, %1, 2;\n\tadd.s64 b, %2, 2;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, 4;\n\tadd.s64 b, %2, 4;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, 6;\n\tadd.s64 b, %2, 6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %4;\n\tadd.s64 b, %2, %5;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %6;\n\tadd.s64 b, %2, %7;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %8;\n\tadd.s64 b, %2, %9;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %10;\n\tadd.s64 b, %2, %11;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(A_PANEL), "n"(B_PANEL), "n"(A_PANEL + 2), "n"(B_PANEL + 2),
        "n"(A_PANEL + 4), "n"(B_PANEL + 4), "n"(A_PANEL + 6), "n"(B_PANEL + 6)
      : "memory");
}
//   tc_mma_ts_x8: D[tmem] (+)= A[tmem] B[smem] over 8 k-steps of 16 keys: A (16-bit P) advances 8 columns per
//   step, B (V, MN-major) B_STEP descriptor units (16 rows of 128 B = 128).  `accumulate` applies to the
//   first step; the rest accumulate.
template <uint32_t B_STEP>
__device__ __forceinline__ void tc_mma_ts_x8(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 b;\n\t.reg .b32 a;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p0;\n\t"
      "add.u32 a, %1, 8;\n\tadd.s64 b, %2, %5;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
      "add.u32 a, %1, 16;\n\tadd.s64 b, %2, %6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
      "add.u32 a, %1, 24;\n\tadd.s64 b, %2, %7;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
      "add.u32 a, %1, 32;\n\tadd.s64 b, %2, %8;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
      "add.u32 a, %1, 40;\n\tadd.s64 b, %2, %9;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
      "add.u32 a, %1, 48;\n\tadd.s64 b, %2, %10;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t"
      "add.u32 a, %1, 56;\n\tadd.s64 b, %2, %11;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [a], b, %3, p1;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "n"(B_STEP), "n"(2 * B_STEP), "n"(3 * B_STEP),
        "n"(4 * B_STEP), "n"(5 * B_STEP), "n"(6 * B_STEP), "n"(7 * B_STEP)
      : "memory");
}
//   tc_mma_ss_pv_x8: D[tmem] (+)= A[smem] B[smem] over 8 k-steps of 16 keys, for O += P V with P in shared
//   memory: A (P, K-major, 128 B rows) advances like the A operand above, B (V, MN-major) B_STEP descriptor
//   units per step.  `accumulate` applies to the first step; the rest accumulate.
template <uint32_t A_PANEL, uint32_t B_STEP>
__device__ __forceinline__ void tc_mma_ss_pv_x8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p0, p1;\n\t.reg .b64 a, b;\n\t"
      "setp.ne.b32 p0, %4, 0;\n\tsetp.eq.b32 p1, %3, %3;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p0;\n\t"
      "add.s64 a, %1, 2;\n\tadd.s64 b, %2, %5;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, 4;\n\tadd.s64 b, %2, %6;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, 6;\n\tadd.s64 b, %2, %7;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %12;\n\tadd.s64 b, %2, %8;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %13;\n\tadd.s64 b, %2, %9;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %14;\n\tadd.s64 b, %2, %10;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t"
      "add.s64 a, %1, %15;\n\tadd.s64 b, %2, %11;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], a, b, %3, p1;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "n"(B_STEP), "n"(2 * B_STEP), "n"(3 * B_STEP),
        "n"(4 * B_STEP), "n"(5 * B_STEP), "n"(6 * B_STEP), "n"(7 * B_STEP), "n"(A_PANEL), "n"(A_PANEL + 2),
        "n"(A_PANEL + 4), "n"(A_PANEL + 6)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// The same wait, naming the registers a preceding tcgen05.ld fills: the load is asynchronous, and the
// in/out operands keep the compiler from moving any use of those registers above the wait.
__device__ __forceinline__ void tc_wait_ld(uint32_t (&r)[32]) {
#if !TB200_PF_TIE
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
  return;
#endif
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
        "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
        "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
        "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :
      : "memory");
}
// Packed pairs of fp32 (sm_100 has two-wide fp32 FMA and ADD on 64-bit register pairs).
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
  return d;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 64-bit shared-memory matrix descriptor, 128B swizzle, version 1 (sm_100).
//   [0,14) start address >> 4 | [16,30) leading byte offset >> 4 | [32,46) stride byte offset >> 4
//   [46,48) version = 1 | [61,64) layout type (2 = SWIZZLE_128B)
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(lbo_bytes >> 4) << 16) |
         (uint64_t(sbo_bytes >> 4) << 32) | (uint64_t(1) << 46) | (uint64_t(2) << 61);
}

// Instruction descriptor of kind::f16: fp32 accumulate, A/B format fmt (0 = f16, 1 = bf16),
// M = 128, N = n, A K-major; B K-major (b_mn = 0) or MN-major (b_mn = 1).
__host__ __device__ constexpr uint32_t make_idesc(uint32_t fmt, uint32_t b_mn, uint32_t n) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn << 16) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}


}  // namespace tb200
