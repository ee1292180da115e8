"""Dispatch keys of the attention slots and the packed-prefill request check
(``src/tileops/ops/attention/selection.py:21-87`` in the reference)."""

from ..kernels.call_spec import AttentionCall, fp8_dtype, uses_sliding_window

__all__ = ["DECODE_KEYS", "DENSE_PREFILL_KEYS", "PACKED_PREFILL_KEYS", "PAGED_DECODE_KEYS",
           "PAGED_DECODE_FP8_KEYS", "PAGED_PREFILL_KEYS", "AttentionCall", "check_packed_prefill_request", "fp8_dtype"]

PACKED_PREFILL_KEYS = (
    "gqa_prefill_fp8_tensor_core_fwd_kernel",
    "gqa_sliding_window_varlen_fwd_kernel",
    "gqa_prefill_square_fwd_kernel",
    "gqa_prefill_causal_fwd_kernel",
    "gqa_prefill_fwd_kernel",
    "gqa_prefill_varlen_fwd_kernel",
)
DENSE_PREFILL_KEYS = ("gqa_prefill_square_fwd_kernel", "gqa_prefill_causal_fwd_kernel", "gqa_prefill_fwd_kernel")
DECODE_KEYS = ("gqa_decode_bs1_kernel", "gqa_decode_kernel")
PAGED_DECODE_KEYS = ("gqa_decode_paged_bs1_kernel", "gqa_decode_paged_kernel")
PAGED_DECODE_FP8_KEYS = ("gqa_decode_paged_fp8_kernel",)
PAGED_PREFILL_KEYS = (
    "gqa_prefill_paged_with_kv_cache_rope_fwd_kernel",
    "gqa_prefill_paged_with_fp8_kv_cache_fwd_kernel",
    "gqa_prefill_paged_with_kv_cache_fwd_kernel",
)


def check_packed_prefill_request(call: AttentionCall) -> None:
    """Reject a packed prefill request that contradicts its ``backend`` parameter."""
    if call.is_fp8:
        if call.backend not in ("auto", "fp8"):
            raise ValueError("FP8 prefill requires backend='auto' or backend='fp8'.")
        if call.is_causal:
            raise ValueError("FP8 prefill currently supports non-causal prefill only.")
        if uses_sliding_window(call):
            raise ValueError("FP8 prefill does not support sliding-window dispatch.")
        if call.max_seqlen_q != call.max_seqlen_kv:
            raise ValueError("FP8 prefill requires max_seqlen_q == max_seqlen_kv.")
        if not call.is_uniform:
            raise ValueError("FP8 prefill requires uniform packed cu_seqlens.")
        return
    if call.backend == "fp8":
        raise ValueError("backend='fp8' requires float8_e4m3fn q/k/v.")
    if uses_sliding_window(call):
        if call.backend not in ("auto", "sliding_window"):
            raise ValueError("sliding-window prefill requires backend='auto' or backend='sliding_window'.")
        return
    if call.backend == "sliding_window":
        raise ValueError("backend='sliding_window' requires window_size_left or window_size_right.")
    if call.backend == "dense" and not call.is_uniform:
        raise ValueError("backend='dense' requires uniform packed cu_seqlens.")
