// Merge of partial attention results over disjoint KV ranges (log2-domain LSE).
//
// The algebra of the reference's split-KV "combine" grid
// (src/tileops/kernels/attention/gqa_decode_paged.py:344-374 in tile-ai/TileOPs), taken one
// level up: the parts come from different GPUs, each holding a slice of every sequence's
// KV cache, and arrive through an all-gather.
#include "tb200_common.cuh"

namespace tb200 {
namespace {

// Arrival flags of a KV-sequence sharded step (flags != null): the parts are written into this GPU's
// memory by the other ranks' decode kernels over NVLink; rank r then stores the step number to
// flags[r] (release, system scope).  Every block waits until all flags have reached the step this
// GPU's own decode kernel just finished (*step_counter), at most wait_cycles clock ticks; on a timeout
// it records code 501 in *status and fills its row with NaN (o) and -inf (lse), so that a step whose
// exchange failed cannot pass for a result.  A block that finds *status already set gives up at once:
// a launch with more rows than resident blocks waits about one limit in total, not one per wave.
// With flags the parts of a step live in the half of the buffers chosen by the step's parity
// (parity_stride floats apart).
template <typename TO>
__global__ void __launch_bounds__(128) lse_merge_kernel(const float* o_parts, const float* lse_parts,
                                                        TO* __restrict__ o, float* __restrict__ lse,
                                                        int parts, int64_t rows, int dim,
                                                        int64_t o_stride, int64_t lse_stride,
                                                        const int* flags, const int* step_counter,
                                                        int64_t parity_stride, int* status,
                                                        long long wait_cycles) {
  const int64_t row = blockIdx.x;
  if (row >= rows) return;
  if (flags) {
    __shared__ int s_ok;
    int step = 0;
    if (threadIdx.x == 0) {
      step = *reinterpret_cast<const volatile int*>(step_counter);
      const long long t0 = clock64();
      int ok = (status && *reinterpret_cast<const volatile int*>(status) != 0) ? 0 : 1;
      for (int r = 0; r < parts && ok; ++r) {
        int seen;
        do {
          asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(flags + r) : "memory");
          if (seen - step >= 0) break;
          if (clock64() - t0 > wait_cycles) { ok = 0; break; }
        } while (true);
      }
      if (!ok && status) atomicCAS(status, 0, 501);
      s_ok = ok ? step + 1 : 0;          // step >= 1, so 0 is free to mean "gave up"
    }
    __syncthreads();
    if (s_ok == 0) {
      for (int d = threadIdx.x; d < dim; d += blockDim.x) store_out<TO>(o + row * dim + d, __int_as_float(0x7fc00000));
      if (lse && threadIdx.x == 0) lse[row] = -INFINITY;
      return;
    }
    const int64_t shift = int64_t((s_ok - 1) & 1) * parity_stride;
    o_parts += shift;
    lse_parts += shift;
  }
  // The LSEs of the first kGroup parts (all of them in the sharded decode, which has at most 8) and this
  // thread's first O values are requested before any is used: one round trip to L2 instead of three.
  constexpr int kGroup = 8;
  float l0[kGroup], x0[kGroup];
  const int d0 = threadIdx.x;
#pragma unroll
  for (int i = 0; i < kGroup; ++i) {
    const bool in = i < parts;
    l0[i] = in ? __ldcg(lse_parts + int64_t(i) * lse_stride + row) : -INFINITY;
    x0[i] = in && d0 < dim ? __ldcg(o_parts + int64_t(i) * o_stride + row * dim + d0) : 0.f;
  }
  float M = kNegFloor;
  bool bad = false;                    // a NaN LSE: that part went wrong, which must not pass for "empty"
#pragma unroll
  for (int i = 0; i < kGroup; ++i) {
    bad |= (l0[i] != l0[i]);
    if (l0[i] > -1e29f) M = fmaxf(M, l0[i]);   // -inf and the finite floor both mean "empty"
  }
  for (int r = kGroup; r < parts; ++r) {
    const float l = __ldcg(lse_parts + int64_t(r) * lse_stride + row);
    bad |= (l != l);
    if (l > -1e29f) M = fmaxf(M, l);
  }
  if (bad) {
    for (int d = threadIdx.x; d < dim; d += blockDim.x) store_out<TO>(o + row * dim + d, __int_as_float(0x7fc00000));
    if (lse && threadIdx.x == 0) lse[row] = __int_as_float(0x7fc00000);
    return;
  }
  float den = 0.f;
  for (int d = d0; d < dim || d == d0; d += blockDim.x) {     // thread 0 always runs once: it owns the LSE
    float acc = 0.f;
    den = 0.f;
#pragma unroll
    for (int i = 0; i < kGroup; ++i) {
      if (l0[i] > -1e29f) {
        const float w = fast_exp2(l0[i] - M);
        den += w;
        acc += w * (d == d0 ? x0[i] : (d < dim ? __ldcg(o_parts + int64_t(i) * o_stride + row * dim + d) : 0.f));
      }
    }
    for (int r = kGroup; r < parts; ++r) {
      const float l = __ldcg(lse_parts + int64_t(r) * lse_stride + row);
      if (l > -1e29f) {
        const float w = fast_exp2(l - M);
        den += w;
        if (d < dim) acc += w * __ldcg(o_parts + int64_t(r) * o_stride + row * dim + d);
      }
    }
    if (d < dim) store_out<TO>(o + row * dim + d, den > 0.f ? acc / den : 0.f);
  }
  if (lse && threadIdx.x == 0) lse[row] = den > 0.f ? M + log2f(den) : -INFINITY;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

namespace {
int merge_impl(const float* o_parts, const float* lse_parts, void* o, float* lse, int parts, int64_t rows, int dim,
               int64_t o_part_stride, int64_t lse_part_stride, int o_dtype, const int* flags,
               const int* step_counter, int64_t parity_stride, int* status, long long wait_cycles, void* stream) {
  if (!o_parts || !lse_parts || !o) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "o_parts, lse_parts and o must be non-null");
  if (parts <= 0 || rows <= 0 || dim <= 0) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "parts, rows and dim must be positive");
  if (o_part_stride == 0) o_part_stride = rows * dim;
  if (lse_part_stride == 0) lse_part_stride = rows;
  if (o_part_stride < rows * dim || lse_part_stride < rows)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "part strides are smaller than one part");
  if (rows > 0x7fffffffLL) TB200_FAIL(TB200_ERR_UNSUPPORTED, "rows exceeds 2^31-1");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const unsigned grid = static_cast<unsigned>(rows);
  switch (o_dtype) {
    case TB200_F32:
      lse_merge_kernel<float><<<grid, 128, 0, s>>>(o_parts, lse_parts, static_cast<float*>(o), lse, parts, rows, dim, o_part_stride, lse_part_stride, flags, step_counter, parity_stride, status, wait_cycles);
      break;
    case TB200_BF16:
      lse_merge_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(o_parts, lse_parts, static_cast<__nv_bfloat16*>(o), lse, parts, rows, dim, o_part_stride, lse_part_stride, flags, step_counter, parity_stride, status, wait_cycles);
      break;
    case TB200_F16:
      lse_merge_kernel<__half><<<grid, 128, 0, s>>>(o_parts, lse_parts, static_cast<__half*>(o), lse, parts, rows, dim, o_part_stride, lse_part_stride, flags, step_counter, parity_stride, status, wait_cycles);
      break;
    default:
      TB200_FAIL(TB200_ERR_UNSUPPORTED, "o_dtype %d is not F16, BF16 or F32", o_dtype);
  }
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}
}  // namespace

extern "C" int tb200_gqa_lse_merge(const float* o_parts, const float* lse_parts, void* o, float* lse,
                                   int parts, int64_t rows, int dim, int64_t o_part_stride,
                                   int64_t lse_part_stride, int o_dtype, void* stream) {
  return merge_impl(o_parts, lse_parts, o, lse, parts, rows, dim, o_part_stride, lse_part_stride, o_dtype, nullptr,
                    nullptr, 0, nullptr, 0, stream);
}

extern "C" int tb200_gqa_lse_merge_wait(const float* o_parts, const float* lse_parts, void* o, float* lse,
                                        int parts, int64_t rows, int dim, int64_t o_part_stride,
                                        int64_t lse_part_stride, int64_t parity_stride, int o_dtype,
                                        const int* flags, const int* step_counter, int* status,
                                        int64_t wait_cycles, void* stream) {
  if (!flags || !step_counter) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "flags and step_counter must be non-null");
  return merge_impl(o_parts, lse_parts, o, lse, parts, rows, dim, o_part_stride, lse_part_stride, o_dtype, flags,
                    step_counter, parity_stride, status, wait_cycles > 0 ? wait_cycles : 1000000000LL, stream);
}
