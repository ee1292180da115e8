"""``tileops.backends`` plugin: the target ``"b200"`` for a TileOPs installation.

A backend plugin registers a device detector and, per operator, a kernel builder
``build_kernel(*TensorSpec, **manifest_params) -> callable`` (``src/tileops/backend/registry.py:42-194``,
``protocol.py:10-53`` of the reference).  This module provides both for the GQA forward family, calling
the sm_100a library through :mod:`tileops_b200.functional`.  The callables take what the operator hands
its kernel (``src/tileops/ops/attention/gqa.py``: packed THD tensors for the prefill ops, the cache and
its metadata for the decode ops).

Packaging (``pyproject.toml`` of the distribution that ships this package)::

    [project.entry-points."tileops.backends"]
    b200 = "tileops_b200.plugin"

Importing the module registers with ``tileops.backend`` when that package is importable (the entry-point
case); :func:`register` does the same with any module exposing ``register_detector`` /
``register_kernel_builder`` (this repository's ``tileops_b200.backend`` in the tests).
"""

from __future__ import annotations

import torch

TARGET = "b200"

__all__ = ["TARGET", "detect", "BUILDERS", "register"]


def detect(device: torch.device) -> bool:
    """True for CUDA devices of compute capability 10.x (B200 / GB200)."""
    if device.type != "cuda" or not torch.cuda.is_available():
        return False
    return torch.cuda.get_device_capability(device)[0] == 10


def _F():
    from . import functional
    return functional


def build_fwd(q, k, v, *, is_causal=True, sm_scale=None, softcap=None, **_):
    """GroupedQueryAttentionFwdOp hands its kernel the packed view of a uniform BSHD batch."""
    B, S, H, D = q.shape
    Hkv = k.shape[2]

    def run(q2, k2, v2, cu_q=None, cu_kv=None, *scales, return_lse=False):
        out = _F().gqa_prefill(q2.view(B, S, H, D), k2.view(B, S, Hkv, D), v2.view(B, S, Hkv, D),
                               is_causal=is_causal, sm_scale=sm_scale, softcap=softcap or 0.0,
                               return_lse=return_lse)
        return (out[0].view(q2.shape), out[1]) if return_lse else out.view(q2.shape)
    return run


def build_packed_prefill(q, k, v, cu_seqlens_q, cu_seqlens_kv, *scales, max_seqlen_q, is_causal=True,
                         sm_scale=None, softcap=None, window_size_left=-1, window_size_right=-1, **_):
    """GroupedQueryAttentionPrefillFwdOp: packed q/k/v with cumulative lengths (uniform or ragged)."""
    def run(q, k, v, cu_q, cu_kv, *scales, return_lse=False):
        return _F().gqa_prefill_paged(q, k, v, None, None, cu_q, None, None, max_seqlen_q,
                                      is_causal=is_causal, sm_scale=sm_scale, softcap=softcap or 0.0,
                                      return_lse=return_lse, cu_seqlens_kv=cu_kv,
                                      window_size_left=window_size_left, window_size_right=window_size_right)
    return run


def build_paged_prefill(q, k_new, v_new, k_pages, v_pages, *rest, page_size, is_causal=True, cache_dtype=None,
                        sm_scale=None, softcap=None, **_):
    """GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp (cache of q's element type)."""
    if k_pages.dtype != q.dtype:
        raise ValueError(f"target {TARGET!r} serves a paged cache of q's element type, got {k_pages.dtype}")

    def run(q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_q, cache_seqlens, block_table,
            max_seqlen_q, cos_table=None, sin_table=None):
        if cos_table is not None or sin_table is not None:
            raise ValueError(f"target {TARGET!r} does not fuse RoPE into the paged prefill")
        return _F().gqa_prefill_paged(q, k_new, v_new, k_pages, v_pages, cu_q, cache_seqlens, block_table,
                                      int(max_seqlen_q), page_size=page_size, is_causal=is_causal,
                                      sm_scale=sm_scale, softcap=softcap or 0.0)
    return run


def build_decode(q, k, v, *, sm_scale=None, softcap=None, **_):
    """GroupedQueryAttentionDecodeWithKVCacheFwdOp: contiguous cache, live length as an argument."""
    def run(q, k, v, real_seqlen_kv=None):
        live = k.shape[1] if real_seqlen_kv is None else real_seqlen_kv
        return _F().gqa_decode(q, k, v, real_seqlen_kv=live, sm_scale=sm_scale, softcap=softcap or 0.0)
    return run


def build_paged_decode(q, k, v, real_seqlen_kv, block_table, *, page_size, sm_scale=None, softcap=None, **_):
    """GroupedQueryAttentionDecodePagedWithKVCacheFwdOp."""
    def run(q, k, v, real_seqlen_kv, block_table):
        return _F().gqa_decode(q, k, v, real_seqlen_kv=real_seqlen_kv, block_table=block_table,
                               page_size=page_size, sm_scale=sm_scale, softcap=softcap or 0.0)
    return run


BUILDERS = {
    "GroupedQueryAttentionFwdOp": build_fwd,
    "GroupedQueryAttentionPrefillFwdOp": build_packed_prefill,
    "GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp": build_paged_prefill,
    "GroupedQueryAttentionDecodeWithKVCacheFwdOp": build_decode,
    "GroupedQueryAttentionDecodePagedWithKVCacheFwdOp": build_paged_decode,
}


def register(backend) -> None:
    """Register the detector and every builder with *backend* (a module or object exposing
    ``register_detector`` and ``register_kernel_builder``)."""
    backend.register_detector(TARGET, detect)
    for op_name, builder in BUILDERS.items():
        backend.register_kernel_builder(op_name, TARGET, builder)


try:  # the entry-point case: a TileOPs installation imports this module to load the target
    import tileops.backend as _tileops_backend
except Exception:  # noqa: BLE001 - no TileOPs here: nothing to register with
    _tileops_backend = None
if _tileops_backend is not None:
    register(_tileops_backend)
