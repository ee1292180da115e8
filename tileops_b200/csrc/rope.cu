// GPT-NeoX rotary embedding of a packed [tokens, heads, dim] tensor at positions given by the
// requests' cached lengths, sm_100a.
//
// Role in the reference: the rotation that GQAPrefillPagedWithKVCacheRopeFwdKernel
// (src/tileops/kernels/attention/gqa_fwd.py:1463-2122 in tile-ai/TileOPs) applies to q and k_new
// before attention and append, with the arithmetic of RopeNeoxPositionIdsFwdOp
// (src/tileops/ops/rope.py:544-640; reference program tests/ops/test_rope.py:84-102): for the
// first rotary_dim dims, split at the midpoint into (x1, x2),
//   y1 = x1 cos - x2 sin,  y2 = x2 cos + x1 sin
// in fp32 with cos / sin tables stored in the tensor's own 16-bit type; the other dims pass through.
// Token t of request b sits at position cache_seqlens[b] + (t - cu_seqlens_q[b]).
//
// HBM bound: every element is read and written once; the tables are small and stay in L2.  Here it
// runs as a pass of its own in front of the tcgen05 prefill kernel: q and k_new of a chunk are a few
// MB, against the cached K/V the prefill then reads.
#include "tb200_common.cuh"

namespace tb200 {
namespace {

template <typename T>
__global__ void __launch_bounds__(128) rope_neox_packed_kernel(
    const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ cos_t, const T* __restrict__ sin_t,
    const int32_t* __restrict__ cu, const int32_t* __restrict__ cache_lens, int batch, int heads, int dim,
    int rotary_dim, int max_position, int* __restrict__ status) {
  const int t = blockIdx.x;
  // request of this token: largest b with cu[b] <= t (batch is small; every thread does the search)
  int lo = 0, hi = batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int pos = (cache_lens ? cache_lens[lo] : 0) + (t - cu[lo]);
  const int half = rotary_dim >> 1;
  const bool pos_ok = pos >= 0 && pos < max_position;
  if (!pos_ok && threadIdx.x == 0 && status) atomicCAS(status, 0, 401);   // reported by the host wrapper
  const T* xt = x + size_t(t) * heads * dim;
  T* yt = y + size_t(t) * heads * dim;
  const T* ct = cos_t + size_t(pos_ok ? pos : 0) * half;
  const T* st = sin_t + size_t(pos_ok ? pos : 0) * half;
  // one thread per (head, pair of the rotated part) and per pass-through element
  const int pairs = heads * half;
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    const float c = float(ct[j]), s = float(st[j]);
    const float x1 = float(xt[h * dim + j]), x2 = float(xt[h * dim + half + j]);
    // unfused multiply and add, as the fp32 reference program rounds them
    yt[h * dim + j] = T(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(-x2, s)));
    yt[h * dim + half + j] = T(__fadd_rn(__fmul_rn(x2, c), __fmul_rn(x1, s)));
  }
  const int rest = dim - rotary_dim;
  for (int i = threadIdx.x; i < heads * rest; i += blockDim.x) {
    const int h = i / rest, j = i - h * rest;
    yt[h * dim + rotary_dim + j] = xt[h * dim + rotary_dim + j];
  }
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_rope_neox_packed(const void* x, void* y, const void* cos_table, const void* sin_table,
                                      const int32_t* cu_seqlens_q, const int32_t* cache_seqlens, int dtype,
                                      int total_tokens, int batch, int heads, int dim, int rotary_dim,
                                      int max_position, int* status, void* stream) {
  if (!x || !y || !cos_table || !sin_table || !cu_seqlens_q)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "x, y, cos_table, sin_table and cu_seqlens_q must be non-null");
  if (total_tokens < 0 || batch <= 0 || heads <= 0 || dim <= 0 || max_position <= 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "batch, heads, dim and max_position must be positive");
  if (rotary_dim <= 0 || rotary_dim > dim || (rotary_dim & 1))
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "rotary_dim must be an even value in (0, dim]");
  if (dtype != TB200_BF16 && dtype != TB200_F16) TB200_FAIL(TB200_ERR_UNSUPPORTED, "dtype must be F16 or BF16");
  if (total_tokens == 0) return TB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == TB200_BF16)
    rope_neox_packed_kernel<__nv_bfloat16><<<total_tokens, 128, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y),
        static_cast<const __nv_bfloat16*>(cos_table), static_cast<const __nv_bfloat16*>(sin_table), cu_seqlens_q,
        cache_seqlens, batch, heads, dim, rotary_dim, max_position, status);
  else
    rope_neox_packed_kernel<__half><<<total_tokens, 128, 0, s>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), static_cast<const __half*>(cos_table),
        static_cast<const __half*>(sin_table), cu_seqlens_q, cache_seqlens, batch, heads, dim, rotary_dim,
        max_position, status);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}
