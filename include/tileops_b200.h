/*
 * tileops_b200 — C ABI of the sm_100a GQA attention-forward kernels.
 *
 * Every entry point takes raw device pointers, plain integers and a CUDA stream
 * (passed as void*, i.e. a cudaStream_t), launches asynchronously on that stream
 * and returns a tb200_status.  Nothing here allocates device memory: callers
 * pass a workspace obtained from the matching *_workspace_bytes() query, zeroed
 * ONCE after allocation (the kernels leave it zeroed again when they finish).
 * No entry point synchronises the host with the device.
 *
 * The functions replace, one for one, the TileLang kernels behind these
 * reference operators (paths relative to the tile-ai/TileOPs tree):
 *   tb200_gqa_decode        GQADecodeKernel.forward        src/tileops/kernels/attention/gqa_decode.py:555-615
 *                           GQADecodePagedKernel.forward   src/tileops/kernels/attention/gqa_decode_paged.py:669-746
 *   tb200_rope_neox_packed  rotation step of GQAPrefillPagedWithKVCacheRopeFwdKernel  src/tileops/kernels/attention/gqa_fwd.py:1463-2122
 *   tb200_gqa_prefill_paged GQAPrefillPagedWithKVCacheFwdKernel  src/tileops/kernels/attention/gqa_fwd.py:600-1002
 *   tb200_gqa_prefill       GQAPrefillFwdKernel / GQAPrefillFwdWsPersistentCausalKernel
 *                                                          src/tileops/kernels/attention/gqa_fwd.py:519-597,
 *                                                          src/tileops/kernels/attention/gqa_prefill_fwd_ws.py:436-520
 *   tb200_gqa_lse_merge     the "combine" grid             src/tileops/kernels/attention/gqa_decode_paged.py:344-374
 *                           (lifted across GPUs; the reference has no multi-GPU form)
 */
#ifndef TILEOPS_B200_H_
#define TILEOPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  TB200_OK = 0,
  TB200_ERR_BAD_ARGUMENT = 1, /* null pointer, non-positive size, heads % heads_kv != 0 ... */
  TB200_ERR_UNSUPPORTED = 2,  /* head dim / dtype combination with no kernel */
  TB200_ERR_WORKSPACE = 3,    /* workspace too small or misaligned */
  TB200_ERR_CUDA = 4,         /* a CUDA runtime call failed; see tb200_last_error() */
  TB200_ERR_TIMEOUT = 5       /* a bounded device-side wait ran out */
} tb200_status;

typedef enum {
  TB200_F16 = 0,
  TB200_BF16 = 1,
  TB200_E4M3 = 2, /* KV cache only */
  TB200_F32 = 3   /* output only */
} tb200_dtype;

/* Human-readable text of the last error raised on the calling thread. */
const char* tb200_last_error(void);

/* Library version, major*100+minor. */
int tb200_version(void);

/* ---------------------------------------------------------------------------
 * Single-token GQA decode over a contiguous or a paged KV cache.
 *
 * Replaces GQADecodeKernel.forward(Q, K, V, real_seqlen_kv:int)
 *   (src/tileops/kernels/attention/gqa_decode.py:555-615) when block_table == NULL, and
 * GQADecodePagedKernel.forward(Q, K, V, real_seqlen_kv, block_table)
 *   (src/tileops/kernels/attention/gqa_decode_paged.py:669-746) otherwise.
 *
 *   q              [batch, heads, dim]            q_dtype (F16 | BF16), contiguous
 *   k, v           paged:      [pool_tokens, heads_kv, dim]
 *                  contiguous: [batch, kv_batch_stride / kv_token_stride tokens, heads_kv, dim]
 *                  kv_dtype == q_dtype, or E4M3 with k_scale / v_scale
 *   o              [batch, heads, dim]            o_dtype (q_dtype | F32), contiguous
 *   lse            [batch, heads] fp32 or NULL    log2-domain: log2(sum_j exp(score_j)); -inf if empty
 *   real_seqlen_kv [batch] int32 device, or NULL -> every sequence has uniform_seqlen tokens
 *   block_table    [batch, block_table_stride] int32 device; logical page i of sequence b is
 *                  physical page block_table[b*stride + i]; only ceil(len_b/page) entries are read
 *   k_scale,v_scale [pool_tokens/page_size, heads_kv] fp32 (E4M3 only): x = float(x_fp8) * scale
 *   kv_token_stride / kv_head_stride / kv_batch_stride: in ELEMENTS of the KV dtype; the last
 *                  dim is contiguous.  kv_batch_stride is used only when block_table == NULL.
 *   sm_scale       multiplies q.k ; softcap > 0 applies cap*tanh(score/cap) before the softmax
 *   kv_pool_tokens token rows behind k / v (paged: rows of the pool; contiguous: ignored, the row
 *                  count per sequence is kv_batch_stride / kv_token_stride).  It bounds what the
 *                  TMA kernel may touch; <= 0 means "not known" (then only the block table bounds it).
 *   flags          0, or an OR of TB200_DECODE_* values (below): the tuning surface that the
 *                  reference exposes as config= / autotune_configs
 *                  (src/tileops/kernels/kernel_base.py:161-202); no environment variable is read.
 *   workspace      tb200_gqa_decode_workspace_bytes(...) bytes, 256-byte aligned, zeroed once.
 *                  The kernel leaves its counters zeroed, so the same buffer serves every later
 *                  call with the SAME (batch, heads, heads_kv, dim); zero it again before using
 *                  it for another shape (the counters then sit elsewhere in the buffer), and
 *                  never share it between launches that may overlap on the GPU.
 *
 * A sequence of length 0 produces a zero output row.  Page ids are not range checked.
 * The kernel never blocks on another CTA: split-KV partials are merged by whichever CTA
 * finishes a (sequence, KV head) last.
 *
 * Two kernels serve this entry point.  Where every 64-token tile is one contiguous piece or two / four
 * whole pages (no block table, page_size a multiple of 64, or page_size 32 / 16), token rows are 128
 * or 256 bytes, q is 16-byte aligned and a KV head has at most 8 q heads, a producer warp streams K/V
 * tiles by TMA ahead of the math warps, across work-item boundaries; every other layout is served by a
 * kernel whose math warps issue cp.async gathers themselves (tb200_gqa_decode_last_kernel tells which).  Waits inside the TMA kernel are bounded (about 0.5 s): if one
 * runs out the launch stops early and the int at byte offset 8 of the workspace is set to a
 * non-zero code (601 producer, 602 math warps); the outputs of that launch are then undefined and
 * the workspace must be zeroed again before its next use.
 * ------------------------------------------------------------------------- */
#define TB200_DECODE_WIDE_ON 1   /* 16-bit cache: force the 3-CTA / 2-stage cp.async kernel (long contexts) */
#define TB200_DECODE_WIDE_OFF 2  /* never pick it */
#define TB200_DECODE_FP8_MMA 4   /* e4m3 cache: e4m3 tensor-core path (page_size % 64 == 0) */
#define TB200_DECODE_NO_TMA 8    /* keep the cp.async kernel where the TMA kernel would apply */
#define TB200_DECODE_CHUNK_TILES_SHIFT 8 /* bits 8..23: fixed split-KV run length in 64-token tiles (0 = cost model) */
#define TB200_DECODE_CHUNK_TILES(n) (((n) & 0xFFFF) << TB200_DECODE_CHUNK_TILES_SHIFT)

size_t tb200_gqa_decode_workspace_bytes(int batch, int heads, int heads_kv, int dim);

int tb200_gqa_decode(const void* q, const void* k, const void* v, void* o, float* lse,
                     const int32_t* real_seqlen_kv, int32_t uniform_seqlen,
                     const int32_t* block_table, int32_t block_table_stride,
                     const float* k_scale, const float* v_scale,
                     int q_dtype, int kv_dtype, int o_dtype,
                     int batch, int heads, int heads_kv, int dim, int page_size,
                     int64_t kv_token_stride, int64_t kv_head_stride, int64_t kv_batch_stride,
                     float sm_scale, float softcap, int64_t kv_pool_tokens, int flags,
                     void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * tb200_gqa_decode for callers that cannot allocate device memory.  (No counterpart in the
 * reference: its kernels allocate their split-KV buffers with torch on every call,
 * src/tileops/kernels/attention/gqa_decode_paged.py:711-721.)
 *
 * Who needs it: a serving runtime that gives the whole device to its own pool allocator at
 * start-up and forbids cudaMalloc afterwards, or a plugin inside another framework whose
 * allocator it may not bypass.  Such a caller has nowhere to get the workspace from, so this
 * variant keeps the split-KV scratch (scheduler counters, merge tickets, fp32 partials) in a
 * fixed array inside the library: TB200_DECODE_STATIC_SCRATCH_BYTES of device memory on every
 * GPU that loads the library, held until the process exits.
 *
 * Arguments and results are those of tb200_gqa_decode without workspace / workspace_bytes; q, k,
 * v, o (and lse, tables, scales) are still the caller's.  The call itself allocates nothing
 * (no cudaMalloc / cudaFree, no allocating library routine): it clears the counters of the
 * shared array with cudaMemsetAsync on `stream` and launches the same kernel.
 *
 *   - A problem whose scratch need (tb200_gqa_decode_workspace_bytes) exceeds
 *     TB200_DECODE_STATIC_SCRATCH_BYTES is refused with TB200_ERR_WORKSPACE and a message
 *     naming both sizes; nothing is launched.
 *   - The first call on each device looks up the array's device address (with that device
 *     current) and loads the kernels; make that first call outside any stream capture.
 *   - All calls on a device share the one array.  Calls that may overlap on the GPU (different
 *     streams, or different host threads) race on it and give wrong results; serialise them on
 *     one stream or use tb200_gqa_decode with separate workspaces.
 * ------------------------------------------------------------------------- */
#define TB200_DECODE_STATIC_SCRATCH_BYTES ((size_t)24 << 20)

int tb200_gqa_decode_noalloc(const void* q, const void* k, const void* v, void* o, float* lse,
                             const int32_t* real_seqlen_kv, int32_t uniform_seqlen,
                             const int32_t* block_table, int32_t block_table_stride,
                             const float* k_scale, const float* v_scale,
                             int q_dtype, int kv_dtype, int o_dtype,
                             int batch, int heads, int heads_kv, int dim, int page_size,
                             int64_t kv_token_stride, int64_t kv_head_stride, int64_t kv_batch_stride,
                             float sm_scale, float softcap, void* stream);

/* ---------------------------------------------------------------------------
 * Merge R partial attention results over disjoint KV ranges (split-KV across GPUs).
 *   o_parts   [R, rows, dim] fp32, each normalised by its own softmax sum; part r starts at
 *             o_parts + r * o_part_stride floats (0 means packed: rows * dim)
 *   lse_parts [R, rows] fp32 log2-domain (-inf or <= -1e29 marks an empty part; a NaN makes the
 *             row's o and lse NaN: a part that went wrong must not pass for an empty one); part r starts
 *             at lse_parts + r * lse_part_stride floats (0 means packed: rows)
 *   o         [rows, dim] o_dtype ; lse [rows] fp32 or NULL
 * Same algebra as the reference's combine grid
 * (src/tileops/kernels/attention/gqa_decode_paged.py:344-374), taken across ranks.
 * ------------------------------------------------------------------------- */
int tb200_gqa_lse_merge(const float* o_parts, const float* lse_parts, void* o, float* lse,
                        int parts, int64_t rows, int dim, int64_t o_part_stride,
                        int64_t lse_part_stride, int o_dtype, void* stream);

/* ---------------------------------------------------------------------------
 * KV-sequence sharded decode across the GPUs of one node, fused with its exchange (no reference
 * counterpart: the reference has no multi-GPU attention; same split-KV algebra as its combine grid,
 * src/tileops/kernels/attention/gqa_decode_paged.py:176-395, taken across ranks).
 *
 * Rank `rank` of `world` (2..8) holds a slice of every sequence's KV.  tb200_gqa_decode_sharded runs the
 * decode kernel on the slice and stores the normalised fp32 partial O and its log2-domain LSE straight
 * into EVERY rank's exchange buffer through peer-mapped pointers (NVLink stores from the decode kernel
 * itself; no collective call), then raises this rank's flag on every rank.  tb200_gqa_lse_merge_wait
 * (next on the same stream) waits for all ranks' flags and merges the parts from local memory.  The wait
 * is bounded: wait_cycles GPU clock ticks (<= 0: about 0.5 s).  When it runs out the kernel records code 501
 * in *status, fills the rows it could not merge with NaN (o) and -inf (lse), and returns; blocks that start
 * after *status is set give up at once, so a launch never waits more than about one limit in total.
 *   peer_buffers[r]: base of rank r's exchange buffer as mapped into this process, 16-byte aligned:
 *       float [2 parities][world slots][batch * heads * (dim + 1)]   (slot = O [batch*heads][dim], then LSE)
 *   peer_flags[r]:   address of this rank's flag word on rank r: int flags[world] on every rank, zeroed
 *       once before the first step; peer_flags[r] = &flags_of_rank_r[rank]
 *   step_counter:    local device int, zeroed once; advanced by every step (a launch reads its step number
 *       and buffer parity from it, so the pair of launches can be replayed from a CUDA graph)
 * All ranks must run the same sequence of steps; consecutive steps alternate the buffer parity, which is
 * enough because a rank cannot start step s + 2 before every rank has merged step s.
 * Merge arguments: o_parts = own buffer base, o_part_stride = slot size in floats,
 * lse_parts = o_parts + batch * heads * dim, lse_part_stride = slot size, parity_stride = world * slot size.
 * ------------------------------------------------------------------------- */
int tb200_gqa_decode_sharded(const void* q, const void* k, const void* v,
                             const int32_t* real_seqlen_kv, int32_t uniform_seqlen,
                             const int32_t* block_table, int32_t block_table_stride,
                             const float* k_scale, const float* v_scale, int q_dtype, int kv_dtype,
                             int batch, int heads, int heads_kv, int dim, int page_size,
                             int64_t kv_token_stride, int64_t kv_head_stride, int64_t kv_batch_stride,
                             float sm_scale, float softcap, int64_t kv_pool_tokens, int flags,
                             void* const* peer_buffers,
                             int* const* peer_flags, int* step_counter, int world, int rank,
                             void* workspace, size_t workspace_bytes, void* stream);

int tb200_gqa_lse_merge_wait(const float* o_parts, const float* lse_parts, void* o, float* lse,
                             int parts, int64_t rows, int dim, int64_t o_part_stride,
                             int64_t lse_part_stride, int64_t parity_stride, int o_dtype,
                             const int* flags, const int* step_counter, int* status,
                             int64_t wait_cycles, void* stream);

/* ---------------------------------------------------------------------------
 * Dense GQA prefill (flash attention forward), BSHD, bottom-right aligned causal mask.
 *
 * Replaces the forward of GQAPrefillFwdKernel (src/tileops/kernels/attention/gqa_fwd.py:519-597)
 * and its Hopper-only specialisations (gqa_prefill_fwd_ws.py:436-520, gqa_fwd_ws.py:1075-1150)
 * for a uniform batch:
 *   q [batch, seqlen_q, heads, dim], k/v [batch, seqlen_kv, heads_kv, dim]  dtype (F16 | BF16)
 *   o [batch, seqlen_q, heads, dim] dtype ; lse [batch, heads, seqlen_q] fp32 log2-domain or NULL
 * dim must be 64, 128 or 256 (tcgen05 path; 256 runs one CTA per SM).  Rows with no visible key give
 * o = 0, lse = -inf.
 * window_left / window_right: sliding window of the reference's
 * GroupedQueryAttentionSlidingWindowFwdOp (src/tileops/ops/attention/gqa.py:1457-1627): with
 * d = seqlen_kv - seqlen_q, key j is visible to row i iff j >= i + d - window_left (when
 * window_left >= 0), j <= i + d + window_right (when window_right >= 0) and j <= i + d (when
 * causal); -1 = unlimited.  Key tiles outside the window of a whole row tile are skipped.
 * flags: 0, or TB200_PREFILL_TWO_TILES to run the kernel with two Q tiles per CTA (head dim 128, dense;
 * measured slower than the default kernel with one Q tile per CTA on B200, kept as a tuning variant): the
 * tuning surface of the reference's config=.
 * workspace: tb200_gqa_prefill_workspace_bytes() bytes, zeroed once.  Its first int is a status word: 0, or
 * the code of a bounded device-side wait that ran out (1xx-3xx, 7xx); once set, later launches return at
 * once with their outputs unwritten until the word is cleared.
 * ------------------------------------------------------------------------- */
#define TB200_PREFILL_TWO_TILES 1

size_t tb200_gqa_prefill_workspace_bytes(int batch, int heads, int heads_kv, int seqlen_q,
                                         int seqlen_kv, int dim);

int tb200_gqa_prefill(const void* q, const void* k, const void* v, void* o, float* lse,
                      int dtype, int batch, int seqlen_q, int seqlen_kv, int heads, int heads_kv,
                      int dim, int is_causal, float sm_scale, float softcap,
                      int window_left, int window_right, int flags,
                      void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * Packed (ragged) GQA prefill of one chunk per request over a paged KV cache, with append.
 *
 * Replaces the forward of GQAPrefillPagedWithKVCacheFwdKernel
 * (src/tileops/kernels/attention/gqa_fwd.py:600-1002; operator
 * GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp, src/tileops/ops/attention/gqa.py:765-1157)
 * and, with the cache arguments NULL, of the packed varlen prefill kernel
 * (src/tileops/kernels/attention/gqa_prefill_varlen_fwd.py; operator
 * GroupedQueryAttentionPrefillVarlenFwdOp, gqa.py:555-762):
 *   q [total_q, heads, dim], k_new / v_new [total_kv, heads_kv, dim]     dtype (F16 | BF16)
 *   cu_seqlens_q [batch + 1] int32: request b owns rows cu[b] .. cu[b+1] of q and o
 *   cu_seqlens_kv [batch + 1] int32: its rows of k_new / v_new; NULL (and total_kv = total_q)
 *   means the same rows as q.  Without a cache the causal mask of a request is bottom-right
 *   aligned: key j is visible to row i iff j <= i + (kv_len - q_len).  With a cache
 *   cu_seqlens_kv must be NULL.
 *   k_pages / v_pages [pool_tokens, heads_kv, dim] dtype, cache_seqlens [batch] int32 (tokens
 *   of request b already cached), block_table [batch, block_table_stride] int32
 *   o [total_q, heads, dim] dtype ; lse [heads, total_q] fp32 log2-domain or NULL
 * Request b attends to its cache_seqlens[b] cached tokens (read from the pages) followed by its
 * own new tokens (read from k_new / v_new): causal means key position <= cache_seqlens[b] + row.
 * The new K/V rows are also written into the pages at logical positions cache_seqlens[b] + i
 * (block_table[b, pos / page_size] * page_size + pos % page_size), in place, by the same launch;
 * cached tokens are never modified.  page_size: a power of two >= 16.  dim: 64, 128 or 256.
 * block_table ids are trusted (range-check them on the host, as the reference operator does).
 * k_pages = v_pages = cache_seqlens = block_table = NULL: no cache, nothing appended.
 * max_seqlen_q bounds the longest request (it sizes the grid).
 * window_left / window_right: as for tb200_gqa_prefill, per request (the reference's
 * GroupedQueryAttentionSlidingWindowVarlenFwdOp, gqa.py:1630-1831); only without a cache.
 * workspace: tb200_gqa_prefill_workspace_bytes() bytes, zeroed once.
 * ------------------------------------------------------------------------- */
int tb200_gqa_prefill_paged(const void* q, const void* k_new, const void* v_new,
                            void* k_pages, void* v_pages, void* o, float* lse,
                            const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_kv,
                            const int32_t* cache_seqlens,
                            const int32_t* block_table, int64_t block_table_stride,
                            int dtype, int total_q, int total_kv, int batch, int max_seqlen_q,
                            int heads, int heads_kv, int dim, int page_size, int64_t pool_tokens,
                            int is_causal, float sm_scale, float softcap,
                            int window_left, int window_right, int flags,
                            void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * Packed prefill of one chunk per request over an FP8-e4m3 paged cache, appending the chunk: ONE launch.
 *
 * Replaces the forward of GQAPrefillPagedWithFP8KVCacheFwdKernel
 * (src/tileops/kernels/attention/gqa_fwd.py:1005-1460; dequantisation at :1059-1065): the kernel of
 * tb200_gqa_prefill_paged reads the e4m3 pages by TMA, four converter warps expand each cached tile in shared
 * memory to the bare e4m3 values in dtype (exact), the tcgen05 MMAs run on the 16-bit tile, the two scalar
 * scales are applied in the softmax (K: to the scores of cached tiles, V: in the exponent of their P; the
 * dequantised values are therefore NOT rounded to dtype first as the reference does - the result is within the
 * operator's tolerance and slightly more accurate), and the appending CTAs quantise the chunk into the pages
 * (x8 = e4m3(x / scale), round to nearest even, saturating at +-448).  An e4m3 NaN code in a page reads as +-480.
 * Measured 20-30 % slower than the three launches below (it converts a tile once per CTA that shares the KV
 * head); it needs no packed 16-bit copy of the cache.
 *   k_pages, v_pages [pool_tokens, heads_kv, dim] e4m3 (modified in place: rows cache_seqlens[b] ...)
 *   k_scale, v_scale  device pointers to ONE fp32 each (the reference keeps one scalar scale per tensor)
 *   every other argument as for tb200_gqa_prefill_paged with a cache; dim must be 128 (other head dims:
 *   tb200_fp8_cache_gather + tb200_gqa_prefill_paged + tb200_fp8_cache_append below)
 * ------------------------------------------------------------------------- */
int tb200_gqa_prefill_paged_e4m3_cache(const void* q, const void* k_new, const void* v_new, void* k_pages,
                                       void* v_pages, const float* k_scale, const float* v_scale, void* o,
                                       float* lse, const int32_t* cu_seqlens_q, const int32_t* cache_seqlens,
                                       const int32_t* block_table, int64_t block_table_stride, int dtype,
                                       int total_q, int batch, int max_seqlen_q, int heads, int heads_kv, int dim,
                                       int page_size, int64_t pool_tokens, int is_causal, float sm_scale,
                                       float softcap, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------
 * GPT-NeoX rotary embedding of a packed tensor at the positions of a prefill chunk.
 *
 * The rotation the reference's fused-RoPE paged prefill applies to q and k_new
 * (GQAPrefillPagedWithKVCacheRopeFwdKernel, src/tileops/kernels/attention/gqa_fwd.py:1463-2122;
 * arithmetic of RopeNeoxPositionIdsFwdOp, src/tileops/ops/rope.py:544-640), as a pass of its own:
 *   x, y [total_tokens, heads, dim] dtype (F16 | BF16), y may not alias x
 *   cos_table, sin_table [max_position, rotary_dim / 2] dtype
 *   token t of request b (cu_seqlens_q[b] <= t < cu_seqlens_q[b+1]) has position
 *   cache_seqlens[b] + t - cu_seqlens_q[b]  (cache_seqlens NULL: 0)
 * The first rotary_dim dims are rotated about their midpoint in fp32, the rest are copied.
 * status: optional device int (zeroed by the caller); set to 401 if a position falls outside
 * [0, max_position) (that token is rotated with position 0).
 * ------------------------------------------------------------------------- */
int tb200_rope_neox_packed(const void* x, void* y, const void* cos_table, const void* sin_table,
                           const int32_t* cu_seqlens_q, const int32_t* cache_seqlens, int dtype,
                           int total_tokens, int batch, int heads, int dim, int rotary_dim,
                           int max_position, int* status, void* stream);

/* ---------------------------------------------------------------------------
 * FP8-e4m3 paged cache with one scalar scale per tensor, around a prefill chunk.
 *
 * Together with tb200_gqa_prefill_paged (no cache, cu_seqlens_kv given) these two replace the forward of
 * GQAPrefillPagedWithFP8KVCacheFwdKernel (src/tileops/kernels/attention/gqa_fwd.py:1005-1460) for head dims
 * other than 128 (head dim 128: tb200_gqa_prefill_paged_e4m3_cache above, one launch):
 *
 * tb200_fp8_cache_gather builds the packed 16-bit K/V the attention reads: for request b, rows
 * cu_seqlens_kv[b] .. +cache_seqlens[b] are its cached tokens dequantised (float(x8) * scale, rounded to
 * dtype), followed by its chunk's own rows of k_new / v_new (copied).
 *   k_pages / v_pages [pool_tokens, heads_kv, dim] e4m3 ; k_new / v_new [total_q, heads_kv, dim] dtype
 *   k_out / v_out [total_kv, heads_kv, dim] dtype, total_kv >= sum_b (cache_seqlens[b] + q_len[b]) (an upper
 *   bound is enough: rows at or behind cu_seqlens_kv[batch] are not touched, so a host that knows only the
 *   capacity of the block table need not read the lengths back)
 *   cu_seqlens_kv [batch + 1] int32 = exclusive sums of cache_seqlens[b] + q_len[b]
 *   k_scale / v_scale: device pointers to one fp32 each
 *
 * tb200_fp8_cache_append writes the chunk into the pages: x8 = e4m3(x / scale), round to nearest even,
 * saturating at +-448, at logical positions cache_seqlens[b] + i.  Cached tokens are not touched.
 * ------------------------------------------------------------------------- */
int tb200_fp8_cache_gather(const void* k_pages, const void* v_pages, const void* k_new, const void* v_new,
                           void* k_out, void* v_out, const int32_t* cu_seqlens_q,
                           const int32_t* cu_seqlens_kv, const int32_t* cache_seqlens,
                           const int32_t* block_table, int64_t block_table_stride,
                           const float* k_scale, const float* v_scale, int dtype, int total_kv,
                           int batch, int heads_kv, int dim, int page_size, void* stream);

int tb200_fp8_cache_append(const void* k_new, const void* v_new, void* k_pages, void* v_pages,
                           const int32_t* cu_seqlens_q, const int32_t* cache_seqlens,
                           const int32_t* block_table, int64_t block_table_stride,
                           const float* k_scale, const float* v_scale, int dtype, int total_q,
                           int batch, int heads_kv, int dim, int page_size, void* stream);

/* ---------------------------------------------------------------------------
 * Tensor-pipe probe (no reference counterpart; a measuring aid of this library).  Every SM runs
 * `repetitions` x 8 tcgen05.mma instructions (cta_group::1, kind::f16, M = 128, K = 16, N = n; A from shared
 * memory, or from TMEM when a_in_tmem != 0) into one accumulator; SM 0 stores into out_clocks[0] the clocks
 * until the last instruction was accepted and into out_clocks[1] the clocks until it completed (-1 if a
 * bounded wait ran out).  Divide by 8 * repetitions for the cost of one instruction.  On B200 it is ~96
 * clocks for n = 64 and n = 128 and 138-171 for n = 256, against 32 / 64 / 128 clocks of arithmetic: the
 * number of MMA instructions per key, not their size, bounds the prefill kernels.
 * ------------------------------------------------------------------------- */
int tb200_mma_issue_probe(int64_t* out_clocks, int n, int a_in_tmem, int repetitions, void* stream);

/* ---------------------------------------------------------------------------
 * Which kernel served the calling thread's last successful tb200_gqa_decode / tb200_gqa_decode_sharded /
 * tb200_gqa_decode_noalloc call (0 before the first).  No reference counterpart: the reference's dispatch
 * reports its choice through `Kernel` objects; here the choice is made inside the library, and tests and
 * benchmarks ask for it to name what they measured.
 * ------------------------------------------------------------------------- */
#define TB200_DECODE_KERNEL_TMA 1       /* gqa_decode_tma_kernel: TMA producer warp + 4 math warps */
#define TB200_DECODE_KERNEL_CP_ASYNC 2  /* gqa_decode_kernel: every thread loads with cp.async */
int tb200_gqa_decode_last_kernel(void);

#ifdef __cplusplus
}
#endif
#endif /* TILEOPS_B200_H_ */
