// Launch parameters and tensor maps shared by the two tcgen05 prefill kernels (gqa_prefill.cu: one
// 128-row Q tile per CTA, two CTAs per SM, every head dim and the packed / paged mode;
// gqa_prefill_pp.cu: two Q tiles per CTA in ping-pong, persistent, dense head dim 128).
#pragma once

#include "tb200_tcgen05.cuh"

namespace tb200 {

constexpr float kRescaleThreshold = 8.f;   // log2 of the growth of the row maximum that forces a rescale
constexpr long long kWaitCycles = 1000000000LL;  // ~0.5 s at 2 GHz

struct PrefillParams {
  void* o;
  float* lse;
  int* status;
  int batch, heads, heads_kv, seqlen_q, seqlen_kv;
  int is_causal;
  int win_left, win_right;     // sliding window around the (bottom-right aligned) diagonal; -1 = unlimited
  float sm_scale, softcap;
  // packed (ragged) queries over a paged cache; unused by the dense kernel
  const int32_t* cu_q;         // [batch + 1] row offsets of the requests in q / o (and k_new / v_new)
  const int32_t* cu_kv;        // [batch + 1] row offsets in k_new / v_new when they differ from cu_q, or null
  const int32_t* cache_lens;   // [batch] tokens already in the pages (null: none)
  const int32_t* bt;           // [batch, bt_stride] logical page -> physical page
  long long bt_stride;
  const void* k_new;           // [total_q, heads_kv, HD]
  const void* v_new;
  void* k_pages;               // [pool_tokens, heads_kv, HD]; null: nothing is appended
  void* v_pages;
  const float* k_scale;        // e4m3 pages (fused variant): one fp32 scale per tensor, on the device
  const float* v_scale;
  int page_size, page_shift, page_box;   // page_box = min(64, page_size): rows per TMA box of the pool maps
  int total_q;
};

// [batch, seq, heads, hd] contiguous 16-bit tensor -> 4-D map (d, head, seq, batch), box 64 x 1 x box_rows x 1
inline int encode_map(CUtensorMap* map, const void* base, int dtype, long long batch, long long seq, int heads, int hd,
             int box_rows) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) TB200_FAIL(TB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[4] = {cuuint64_t(hd), cuuint64_t(heads), cuuint64_t(seq), cuuint64_t(batch)};
  cuuint64_t strides[3] = {cuuint64_t(hd) * 2, cuuint64_t(heads) * hd * 2, cuuint64_t(seq) * heads * hd * 2};
  cuuint32_t box[4] = {64, 1, cuuint32_t(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, dtype == TB200_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B,
                   hd * 2 >= 256 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,   // a head's row
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) TB200_FAIL(TB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  return TB200_OK;
}

// Encoding a map is a driver call (microseconds on the host); a serving loop presents the same pools, and
// often the same q / k_new / v_new staging buffers, call after call, so the last few maps are kept per thread.
inline int make_map(CUtensorMap* map, const void* base, int dtype, long long batch, long long seq, int heads, int hd,
                    int box_rows) {
  struct Key {
    const void* base; int dtype, heads, hd, box_rows; long long batch, seq;
    bool operator==(const Key& o) const {
      return base == o.base && dtype == o.dtype && heads == o.heads && hd == o.hd && box_rows == o.box_rows &&
             batch == o.batch && seq == o.seq;
    }
  };
  constexpr int kSlots = 16;
  struct Slot { Key key; CUtensorMap map; bool used; };
  static thread_local Slot cache[kSlots] = {};
  static thread_local int next = 0;
  const Key key{base, dtype, heads, hd, box_rows, batch, seq};
  for (int i = 0; i < kSlots; ++i)
    if (cache[i].used && cache[i].key == key) { *map = cache[i].map; return TB200_OK; }
  const int st = encode_map(map, base, dtype, batch, seq, heads, hd, box_rows);
  if (st != TB200_OK) return st;
  cache[next] = Slot{key, *map, true};
  next = (next + 1) % kSlots;
  return TB200_OK;
}

// e4m3 pool [tokens, heads, hd] (one byte per element) -> 4-D map (d, head, token, 1), box hd bytes x 1 x box_rows x 1
// (hd = 128: one 128-byte swizzled row per token, the layout the converter warps of the fused kernel expand in place)
inline int make_map_e4m3(CUtensorMap* map, const void* base, long long tokens, int heads, int hd, int box_rows) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (!enc) TB200_FAIL(TB200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[4] = {cuuint64_t(hd), cuuint64_t(heads), cuuint64_t(tokens), 1};
  cuuint64_t strides[3] = {cuuint64_t(hd), cuuint64_t(heads) * hd, cuuint64_t(tokens) * heads * hd};
  cuuint32_t box[4] = {cuuint32_t(hd), 1, cuuint32_t(box_rows), 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) TB200_FAIL(TB200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", int(r));
  return TB200_OK;
}

struct PrefillMaps {
  CUtensorMap q, k, v, kp, vp;
};


// Defined in gqa_prefill_pp.cu: TB200_OK after launching, kPrefillPpNotApplicable when that kernel does
// not serve the call (the caller then launches the kernel of gqa_prefill.cu), or an error.
constexpr int kPrefillPpNotApplicable = -1;
int launch_prefill_pp(const PrefillMaps& m, const PrefillParams& p, int dtype, int head_dim, bool paged,
                      cudaStream_t stream);

}  // namespace tb200
