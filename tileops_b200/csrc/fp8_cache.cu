// FP8-e4m3 paged KV cache with ONE scalar scale per tensor, as the reference's paged prefill keeps
// it, sm_100a: the two data movements around the attention of a prefill chunk.
//
// Role in the reference: GQAPrefillPagedWithFP8KVCacheFwdKernel
// (src/tileops/kernels/attention/gqa_fwd.py:1005-1460 in tile-ai/TileOPs) dequantises the cached
// pages on the fly (x = float(x8) * scale, rounded to the attention type), attends to them and to
// the chunk's own full-precision k_new / v_new, and appends the chunk quantised
// (x8 = e4m3(x / scale)).  Here the tcgen05 attention kernel takes 16-bit operands, so the cached
// tokens are first gathered and dequantised into a packed 16-bit K/V next to the chunk's own rows
// (tb200_fp8_cache_gather), the packed varlen prefill runs on that, and the chunk is quantised into
// the pages (tb200_fp8_cache_append).  Both kernels are HBM bound: one read and one write per element.
//
// Conversion: round to nearest even; values beyond +-448 saturate to +-448 (the reference's torch cast
// turns them into NaN; in-range values are bit-identical).
#include <cuda_fp8.h>

#include "tb200_common.cuh"

namespace tb200 {
namespace {

constexpr int kThreads = 128;

__device__ __forceinline__ int find_request(const int32_t* cu, int batch, int t) {
  int lo = 0, hi = batch - 1;   // largest b with cu[b] <= t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float e4m3_to_float(unsigned char b) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(b, __NV_E4M3);
  return __half2float(__half(hr));
}
__device__ __forceinline__ unsigned char float_to_e4m3(float x) {
  return __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}

// One block per token of the packed [old | new] K/V of all requests.
template <typename T>
__global__ void __launch_bounds__(kThreads) fp8_cache_gather_kernel(
    const unsigned char* __restrict__ k_pages, const unsigned char* __restrict__ v_pages,
    const T* __restrict__ k_new, const T* __restrict__ v_new, T* __restrict__ k_out, T* __restrict__ v_out,
    const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_kv, const int32_t* __restrict__ cache_lens,
    const int32_t* __restrict__ bt, long long bt_stride, const float* __restrict__ k_scale,
    const float* __restrict__ v_scale, int batch, int row_elems, int page_size) {
  const int g = blockIdx.x;
  if (g >= cu_kv[batch]) return;        // total_kv may be an upper bound (the host never reads the lengths)
  const int b = find_request(cu_kv, batch, g);
  const int t = g - cu_kv[b];
  const int old = cache_lens[b];
  T* ko = k_out + size_t(g) * row_elems;
  T* vo = v_out + size_t(g) * row_elems;
  if (t < old) {
    const int page = bt[(long long)b * bt_stride + t / page_size];
    const size_t src = (size_t(page) * page_size + t % page_size) * row_elems;
    const float ks = *k_scale, vs = *v_scale;
    if (row_elems % 8 == 0) {           // 8 elements per step: 8-byte loads, 16-byte stores (rows are 8-element aligned)
      for (int i = threadIdx.x * 8; i < row_elems; i += kThreads * 8) {
        alignas(8) unsigned char kb[8], vb[8];
        alignas(16) T kq[8], vq[8];
        *reinterpret_cast<uint2*>(kb) = *reinterpret_cast<const uint2*>(k_pages + src + i);
        *reinterpret_cast<uint2*>(vb) = *reinterpret_cast<const uint2*>(v_pages + src + i);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          kq[e] = T(e4m3_to_float(kb[e]) * ks);
          vq[e] = T(e4m3_to_float(vb[e]) * vs);
        }
        *reinterpret_cast<uint4*>(ko + i) = *reinterpret_cast<const uint4*>(kq);
        *reinterpret_cast<uint4*>(vo + i) = *reinterpret_cast<const uint4*>(vq);
      }
    } else {
      for (int i = threadIdx.x; i < row_elems; i += kThreads) {
        ko[i] = T(e4m3_to_float(k_pages[src + i]) * ks);
        vo[i] = T(e4m3_to_float(v_pages[src + i]) * vs);
      }
    }
  } else {
    const size_t src = size_t(cu_q[b] + t - old) * row_elems;
    if (row_elems % 8 == 0) {
      for (int i = threadIdx.x * 8; i < row_elems; i += kThreads * 8) {
        *reinterpret_cast<uint4*>(ko + i) = *reinterpret_cast<const uint4*>(k_new + src + i);
        *reinterpret_cast<uint4*>(vo + i) = *reinterpret_cast<const uint4*>(v_new + src + i);
      }
    } else {
      for (int i = threadIdx.x; i < row_elems; i += kThreads) {
        ko[i] = k_new[src + i];
        vo[i] = v_new[src + i];
      }
    }
  }
}

// One block per new token: quantise its K and V rows into the pages.
template <typename T>
__global__ void __launch_bounds__(kThreads) fp8_cache_append_kernel(
    const T* __restrict__ k_new, const T* __restrict__ v_new, unsigned char* __restrict__ k_pages,
    unsigned char* __restrict__ v_pages, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cache_lens,
    const int32_t* __restrict__ bt, long long bt_stride, const float* __restrict__ k_scale,
    const float* __restrict__ v_scale, int batch, int row_elems, int page_size) {
  const int t = blockIdx.x;
  const int b = find_request(cu_q, batch, t);
  const int pos = cache_lens[b] + t - cu_q[b];
  const int page = bt[(long long)b * bt_stride + pos / page_size];
  const size_t dst = (size_t(page) * page_size + pos % page_size) * row_elems;
  const size_t src = size_t(t) * row_elems;
  const float ks = *k_scale, vs = *v_scale;
  if (row_elems % 8 == 0) {
    for (int i = threadIdx.x * 8; i < row_elems; i += kThreads * 8) {
      alignas(16) T kq[8], vq[8];
      alignas(8) unsigned char kb[8], vb[8];
      *reinterpret_cast<uint4*>(kq) = *reinterpret_cast<const uint4*>(k_new + src + i);
      *reinterpret_cast<uint4*>(vq) = *reinterpret_cast<const uint4*>(v_new + src + i);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        kb[e] = float_to_e4m3(__fdiv_rn(float(kq[e]), ks));
        vb[e] = float_to_e4m3(__fdiv_rn(float(vq[e]), vs));
      }
      *reinterpret_cast<uint2*>(k_pages + dst + i) = *reinterpret_cast<const uint2*>(kb);
      *reinterpret_cast<uint2*>(v_pages + dst + i) = *reinterpret_cast<const uint2*>(vb);
    }
  } else {
    for (int i = threadIdx.x; i < row_elems; i += kThreads) {
      k_pages[dst + i] = float_to_e4m3(__fdiv_rn(float(k_new[src + i]), ks));
      v_pages[dst + i] = float_to_e4m3(__fdiv_rn(float(v_new[src + i]), vs));
    }
  }
}

int check_common(const void* a, const void* b, const void* c, const void* d, int dtype, int batch, int heads_kv,
                 int dim, int page_size) {
  if (!a || !b || !c || !d) TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "tensor arguments must be non-null");
  if (dtype != TB200_BF16 && dtype != TB200_F16) TB200_FAIL(TB200_ERR_UNSUPPORTED, "dtype must be F16 or BF16");
  if (batch <= 0 || heads_kv <= 0 || dim <= 0 || page_size <= 0)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "batch, heads_kv, dim and page_size must be positive");
  return TB200_OK;
}

}  // namespace
}  // namespace tb200

using namespace tb200;

extern "C" int tb200_fp8_cache_gather(const void* k_pages, const void* v_pages, const void* k_new, const void* v_new,
                                      void* k_out, void* v_out, const int32_t* cu_seqlens_q,
                                      const int32_t* cu_seqlens_kv, const int32_t* cache_seqlens,
                                      const int32_t* block_table, int64_t block_table_stride, const float* k_scale,
                                      const float* v_scale, int dtype, int total_kv, int batch, int heads_kv, int dim,
                                      int page_size, void* stream) {
  int st = check_common(k_pages, v_pages, k_new, v_new, dtype, batch, heads_kv, dim, page_size);
  if (st != TB200_OK) return st;
  if (!k_out || !v_out || !cu_seqlens_q || !cu_seqlens_kv || !cache_seqlens || !block_table || !k_scale || !v_scale)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "outputs, length tensors, block_table and scales must be non-null");
  if (total_kv <= 0) return TB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int row = heads_kv * dim;
  auto kp = static_cast<const unsigned char*>(k_pages), vp = static_cast<const unsigned char*>(v_pages);
  if (dtype == TB200_BF16)
    fp8_cache_gather_kernel<__nv_bfloat16><<<total_kv, kThreads, 0, s>>>(
        kp, vp, static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new),
        static_cast<__nv_bfloat16*>(k_out), static_cast<__nv_bfloat16*>(v_out), cu_seqlens_q, cu_seqlens_kv,
        cache_seqlens, block_table, block_table_stride, k_scale, v_scale, batch, row, page_size);
  else
    fp8_cache_gather_kernel<__half><<<total_kv, kThreads, 0, s>>>(
        kp, vp, static_cast<const __half*>(k_new), static_cast<const __half*>(v_new), static_cast<__half*>(k_out),
        static_cast<__half*>(v_out), cu_seqlens_q, cu_seqlens_kv, cache_seqlens, block_table, block_table_stride,
        k_scale, v_scale, batch, row, page_size);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}

extern "C" int tb200_fp8_cache_append(const void* k_new, const void* v_new, void* k_pages, void* v_pages,
                                      const int32_t* cu_seqlens_q, const int32_t* cache_seqlens,
                                      const int32_t* block_table, int64_t block_table_stride, const float* k_scale,
                                      const float* v_scale, int dtype, int total_q, int batch, int heads_kv, int dim,
                                      int page_size, void* stream) {
  int st = check_common(k_new, v_new, k_pages, v_pages, dtype, batch, heads_kv, dim, page_size);
  if (st != TB200_OK) return st;
  if (!cu_seqlens_q || !cache_seqlens || !block_table || !k_scale || !v_scale)
    TB200_FAIL(TB200_ERR_BAD_ARGUMENT, "length tensors, block_table and scales must be non-null");
  if (total_q <= 0) return TB200_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int row = heads_kv * dim;
  auto kp = static_cast<unsigned char*>(k_pages), vp = static_cast<unsigned char*>(v_pages);
  if (dtype == TB200_BF16)
    fp8_cache_append_kernel<__nv_bfloat16><<<total_q, kThreads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new), kp, vp, cu_seqlens_q,
        cache_seqlens, block_table, block_table_stride, k_scale, v_scale, batch, row, page_size);
  else
    fp8_cache_append_kernel<__half><<<total_q, kThreads, 0, s>>>(
        static_cast<const __half*>(k_new), static_cast<const __half*>(v_new), kp, vp, cu_seqlens_q, cache_seqlens,
        block_table, block_table_stride, k_scale, v_scale, batch, row, page_size);
  TB200_CUDA_CHECK(cudaGetLastError());
  return TB200_OK;
}
