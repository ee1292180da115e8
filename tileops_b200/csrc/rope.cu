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

// Vector form for rotary_dim % 16 == 0 and dim % 8 == 0: a work item is 8 consecutive elements
// (16 bytes) of one (token, head).  An item in the first half of the rotated part loads its partner
// 8 elements from the second half and writes both results; an item of the second half has nothing
// to do; an item behind the rotated part is a 16-byte copy.
template <typename T>
__global__ void __launch_bounds__(128) rope_neox_packed_vec8_kernel(
    const T* __restrict__ x, T* __restrict__ y, const T* __restrict__ cos_t, const T* __restrict__ sin_t,
    const int32_t* __restrict__ cu, const int32_t* __restrict__ cache_lens, int batch, int heads, int dim,
    int rotary_dim, int max_position, int* __restrict__ status) {
  const int t = blockIdx.x;
  int lo = 0, hi = batch - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int pos = (cache_lens ? cache_lens[lo] : 0) + (t - cu[lo]);
  const int half = rotary_dim >> 1;
  const bool pos_ok = pos >= 0 && pos < max_position;
  if (!pos_ok && threadIdx.x == 0 && status) atomicCAS(status, 0, 401);
  const T* xt = x + size_t(t) * heads * dim;
  T* yt = y + size_t(t) * heads * dim;
  const T* ct = cos_t + size_t(pos_ok ? pos : 0) * half;
  const T* st = sin_t + size_t(pos_ok ? pos : 0) * half;
  const int per_head = dim >> 3;
  for (int i = threadIdx.x; i < heads * per_head; i += blockDim.x) {
    const int h = i / per_head, j0 = (i - h * per_head) << 3;
    const T* xr = xt + h * dim;
    T* yr = yt + h * dim;
    if (j0 >= rotary_dim) {
      *reinterpret_cast<uint4*>(yr + j0) = *reinterpret_cast<const uint4*>(xr + j0);
    } else if (j0 < half) {
      alignas(16) T a[8], b[8], c[8], sn[8], o1[8], o2[8];
      *reinterpret_cast<uint4*>(a) = *reinterpret_cast<const uint4*>(xr + j0);
      *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(xr + half + j0);
      *reinterpret_cast<uint4*>(c) = *reinterpret_cast<const uint4*>(ct + j0);
      *reinterpret_cast<uint4*>(sn) = *reinterpret_cast<const uint4*>(st + j0);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x1 = float(a[e]), x2 = float(b[e]), cc = float(c[e]), ss = float(sn[e]);
        o1[e] = T(__fadd_rn(__fmul_rn(x1, cc), __fmul_rn(-x2, ss)));
        o2[e] = T(__fadd_rn(__fmul_rn(x2, cc), __fmul_rn(x1, ss)));
      }
      *reinterpret_cast<uint4*>(yr + j0) = *reinterpret_cast<const uint4*>(o1);
      *reinterpret_cast<uint4*>(yr + half + j0) = *reinterpret_cast<const uint4*>(o2);
    }
  }
}

template <typename T>
void launch_rope(const void* x, void* y, const void* c, const void* sn, const int32_t* cu, const int32_t* cache,
                 int total, int batch, int heads, int dim, int rotary_dim, int max_position, int* status,
                 cudaStream_t s) {
  const bool vec = rotary_dim % 16 == 0 && dim % 8 == 0 &&
                   ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) | reinterpret_cast<uintptr_t>(c) |
                     reinterpret_cast<uintptr_t>(sn)) & 15) == 0;
  auto kern = vec ? rope_neox_packed_vec8_kernel<T> : rope_neox_packed_kernel<T>;
  kern<<<total, 128, 0, s>>>(static_cast<const T*>(x), static_cast<T*>(y), static_cast<const T*>(c),
                             static_cast<const T*>(sn), cu, cache, batch, heads, dim, rotary_dim, max_position,
                             status);
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
    launch_rope<__nv_bfloat16>(x, y, cos_table, sin_table, cu_seqlens_q, cache_seqlens, total_tokens, batch, heads,
                               dim, rotary_dim, max_position, status, s);
  else
    launch_rope<__half>(x, y, cos_table, sin_table, cu_seqlens_q, cache_seqlens, total_tokens, batch, heads, dim,
                        rotary_dim, max_position, status, s);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}
