// Merge of partial attention results over disjoint KV ranges (log2-domain LSE).
//
// The algebra of the reference's split-KV "combine" grid
// (src/tileops/kernels/attention/gqa_decode_paged.py:344-374 in tile-ai/TileOPs), taken one
// level up: the parts come from different GPUs, each holding a slice of every sequence's
// KV cache, and arrive through an all-gather.
#include "tb200_common.cuh"

namespace tb200 {
namespace {

template <typename TO>
__global__ void __launch_bounds__(128) lse_merge_kernel(const float* __restrict__ o_parts,
                                                        const float* __restrict__ lse_parts,
                                                        TO* __restrict__ o, float* __restrict__ lse,
                                                        int parts, int64_t rows, int dim,
                                                        int64_t o_stride, int64_t lse_stride) {
  const int64_t row = blockIdx.x;
  if (row >= rows) return;
  float M = kNegFloor;
  for (int r = 0; r < parts; ++r) {
    float l = lse_parts[int64_t(r) * lse_stride + row];
    if (l > -1e29f) M = fmaxf(M, l);   // -inf and the finite floor both mean "empty"
  }
  float den = 0.f;
  for (int r = 0; r < parts; ++r) {
    float l = lse_parts[int64_t(r) * lse_stride + row];
    if (l > -1e29f) den += fast_exp2(l - M);
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < parts; ++r) {
      float l = lse_parts[int64_t(r) * lse_stride + row];
      if (l > -1e29f) acc += fast_exp2(l - M) * o_parts[int64_t(r) * o_stride + row * dim + d];
    }
    store_out<TO>(o + row * dim + d, acc * inv);
  }
  if (lse && threadIdx.x == 0) lse[row] = den > 0.f ? M + log2f(den) : -INFINITY;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_gqa_lse_merge(const float* o_parts, const float* lse_parts, void* o, float* lse,
                                   int parts, int64_t rows, int dim, int64_t o_part_stride,
                                   int64_t lse_part_stride, int o_dtype, void* stream) {
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
      lse_merge_kernel<float><<<grid, 128, 0, s>>>(o_parts, lse_parts, static_cast<float*>(o), lse, parts, rows, dim, o_part_stride, lse_part_stride);
      break;
    case TB200_BF16:
      lse_merge_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(o_parts, lse_parts, static_cast<__nv_bfloat16*>(o), lse, parts, rows, dim, o_part_stride, lse_part_stride);
      break;
    case TB200_F16:
      lse_merge_kernel<__half><<<grid, 128, 0, s>>>(o_parts, lse_parts, static_cast<__half*>(o), lse, parts, rows, dim, o_part_stride, lse_part_stride);
      break;
    default:
      TB200_FAIL(TB200_ERR_UNSUPPORTED, "o_dtype %d is not F16, BF16 or F32", o_dtype);
  }
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}
