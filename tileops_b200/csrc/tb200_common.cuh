// Shared host/device helpers for the tileops_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "tileops_b200.h"

namespace tb200 {

// ---- host-side error text (per thread) -------------------------------------------------
char* error_buffer();  // 512 bytes, thread local (defined in tb200_common.cu)

#define TB200_FAIL(code, ...)                                   \
  do {                                                          \
    snprintf(::tb200::error_buffer(), 512, __VA_ARGS__);        \
    return (code);                                              \
  } while (0)

#define TB200_CUDA_CHECK(expr)                                                        \
  do {                                                                                \
    cudaError_t _e = (expr);                                                          \
    if (_e != cudaSuccess)                                                            \
      TB200_FAIL(TB200_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e));     \
  } while (0)

int sm_count();  // multiprocessors of the current device (cached per device)

// ---- device helpers ---------------------------------------------------------------------
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kNegFloor = -1.0e30f;  // finite stand-in for "no key seen yet"

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}

// D(16x8,f32) += A(16x16) * B(16x8)
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4],
                                                         const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4],
                                                  const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}


// D(16x8,f32) += A(16x32, e4m3) * B(32x8, e4m3)
__device__ __forceinline__ void mma_16832_e4m3(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Two floats -> two e4m3 bytes (round to nearest, saturating): byte 0 = lo, byte 1 = hi.
__device__ __forceinline__ uint32_t f32x2_to_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;\n" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
// Two e4m3 bytes (byte 0, byte 1 of the low half of x) -> two floats.
__device__ __forceinline__ float2 e4m3x2_to_f32x2(uint32_t x) {
  uint32_t h;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;\n" : "=r"(h) : "h"(uint16_t(x)));
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}
// A value as the sum of two e4m3 numbers: hi = rn(x), lo = rn(x - hi); returns bytes (hi0, hi1) and
// (lo0, lo1) for the pair (x0, x1).  With |x| <= 448 the pair carries about 8 significant bits.
__device__ __forceinline__ void split_e4m3x2(float x0, float x1, uint32_t& hi, uint32_t& lo) {
  hi = f32x2_to_e4m3x2(x0, x1);
  const float2 h = e4m3x2_to_f32x2(hi);
  lo = f32x2_to_e4m3x2(x0 - h.x, x1 - h.y);
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t y;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(y) : "r"(a), "r"(b), "r"(sel));
  return y;
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// The two 16-bit values of a register as floats (inverse of pack2).
template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t x);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t x) {
  return make_float2(__uint_as_float(x << 16), __uint_as_float(x & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t x) {
  return __half22float2(*reinterpret_cast<const __half2*>(&x));
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
// Two exponentials per MUFU instruction: the pair is rounded to f16 (11 significant bits: for |x| < 8
// an absolute error below 2^-8 in x, i.e. below 0.3 % in 2^x), and 2^x comes back as an f16 pair.
// -inf and anything below the f16 range give +0.
__device__ __forceinline__ uint32_t f32x2_to_f16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}
__device__ __forceinline__ uint32_t ex2_f16x2(uint32_t x) {
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t add_f16x2(uint32_t a, uint32_t b) {
  uint32_t y;
  asm("add.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
  return y;
}
__device__ __forceinline__ float2 f16x2_to_f32x2(uint32_t h) {
  return __half22float2(*reinterpret_cast<__half2*>(&h));
}
// 2^x on the FMA and integer pipes (no MUFU): floor by a round-down add of 1.5*2^23, a cubic for
// 2^frac on [0,1), then the integer part is added to the exponent field.  Relative error about
// 1e-4 (well under bf16 resolution).  x is clamped at -127, so very negative inputs (and -inf)
// give about 6e-39 instead of 0: use it only where every input is finite.
__device__ __forceinline__ float exp2_poly(float x) {
  x = fmaxf(x, -127.f);
  float xr;
  asm("add.rm.f32 %0, %1, %2;\n" : "=f"(xr) : "f"(x), "f"(12582912.f));
  const float f = x - (xr - 12582912.f);
  float p = fmaf(f, 0.07711909f, 0.22756439f);
  p = fmaf(p, f, 0.69514614f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(xr) << 23));
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float y;
  asm("max.f32 %0, %1, %2, %3;\n" : "=f"(y) : "f"(a), "f"(b), "f"(c));
  return y;
}
__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// Two e4m3 bytes of `x` (selected by the PRMT selector SEL, which must place them in bytes 1
// and 3 of the result and zero in bytes 0 and 2) -> packed f16x2 holding kE4m3Unit^-1 times their
// values.
//   TB200_FP8_CVT=0: integer path.  Moving the 7 magnitude bits one place down turns the e4m3
//     exponent/mantissa into an f16 exponent/mantissa with the bias off by 8 (subnormals
//     included); the sign is carried from bit 14 into bit 15 by adding bit 14 to itself.  Result
//     is 2^-8 times the value (kE4m3Unit = 256).
//   TB200_FP8_CVT=1: the hardware conversion cvt.rn.f16x2.e4m3x2 (exact values, kE4m3Unit = 1).
#ifndef TB200_FP8_CVT
#define TB200_FP8_CVT 1
#endif
#if TB200_FP8_CVT
constexpr float kE4m3Unit = 1.f;
#else
constexpr float kE4m3Unit = 256.f;
#endif
template <uint32_t SEL>
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2_scaled(uint32_t x) {
#if TB200_FP8_CVT
  // SEL names the two source bytes in its nibbles 1 and 3; gather them into the low half
  uint32_t h;
  if constexpr (SEL == 0x1404u) {          // bytes 0,1: the low half as it is
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(h) : "r"(x));
  } else if constexpr (SEL == 0x3424u) {   // bytes 2,3: the high half as it is
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, hi;\n\t}" : "=r"(h) : "r"(x));
  } else {
    constexpr uint32_t sel2 = ((SEL >> 4) & 0xF) | (((SEL >> 12) & 0xF) << 4) | 0x4400u;
    uint32_t y;
    asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(y) : "r"(x), "r"(0u), "n"(sel2));
    asm("{\n\t.reg .b16 lo, hi;\n\tmov.b32 {lo, hi}, %1;\n\tcvt.rn.f16x2.e4m3x2 %0, lo;\n\t}" : "=r"(h) : "r"(y));
  }
  return h;
#else
  uint32_t y;
  asm("prmt.b32 %0, %1, %2, %3;\n" : "=r"(y) : "r"(x), "r"(0u), "n"(SEL));
  uint32_t t = y >> 1;
  return t + (t & 0x40004000u);
#endif
}

template <typename T>
__device__ __forceinline__ void store_out(T* p, float v);
template <>
__device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_out<__nv_bfloat16>(__nv_bfloat16* p, float v) {
  *p = __float2bfloat16_rn(v);
}
template <>
__device__ __forceinline__ void store_out<__half>(__half* p, float v) { *p = __float2half_rn(v); }

}  // namespace tb200
