"""sm_100a kernel class for dense GQA prefill (L1 of the operator stack).

Replaces, in the ``gqa_prefill_fwd_kernel`` slot, the reference's ``GQAPrefillFwdKernel``
(``src/tileops/kernels/attention/gqa_fwd.py:519-597``) and stands in for its two Hopper-only
specialisations (``gqa_prefill_fwd_ws.py:436``, ``gqa_fwd_ws.py:1075``), none of which runs on
sm_100.  Keyword constructor and packed ``forward`` follow the reference
(``src/tileops/ops/attention/gqa.py:113-128``, ``kernels/attention/packed_prefill.py:71-83``):
the packed THD tensors of a uniform batch are viewed as BSHD and handed to the tcgen05 kernel
through the C ABI (``tb200_gqa_prefill``).
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import functional as F
from .call_spec import ATTENTION_DTYPES, dense_prefill_region
from .kernel_base import Kernel

_PREFILL_DIMS = (64, 128, 256)   # head dims the tcgen05 prefill kernel is instantiated for

__all__ = ["GQAPrefillSm100Kernel", "GQAPrefillVarlenSm100Kernel", "GQAPrefillPagedSm100Kernel",
           "GQASlidingWindowSm100Kernel", "GQASlidingWindowVarlenSm100Kernel", "GQAPrefillPagedRopeSm100Kernel", "GQAPrefillPagedFp8CacheSm100Kernel"]


class GQAPrefillSm100Kernel(Kernel):
    supported_archs = [100]
    general = True

    @classmethod
    def applies(cls, call) -> bool:
        return dense_prefill_region(call) and call.dim in _PREFILL_DIMS and call.dtype in ATTENTION_DTYPES

    def __init__(self, batch, heads, heads_kv, max_seqlen_q, max_seqlen_kv, dim, is_causal, dtype,
                 sm_scale=None, softcap=0.0, window_size_left=-1, window_size_right=-1,
                 accum_dtype=torch.float32, config: Optional[dict] = None, tune: bool = False,
                 device_index=None) -> None:
        super().__init__(device_index=device_index)
        if dim not in _PREFILL_DIMS:
            raise ValueError(f"GQAPrefillSm100Kernel supports head dim 64, 128 and 256, got {dim}")
        self.window_size_left, self.window_size_right = window_size_left, window_size_right
        self.batch, self.heads, self.heads_kv, self.dim = batch, heads, heads_kv, dim
        self.max_seqlen_q, self.max_seqlen_kv = max_seqlen_q, max_seqlen_kv
        self.is_causal, self.dtype = is_causal, dtype
        self.sm_scale = dim ** -0.5 if sm_scale is None else sm_scale
        self.softcap = 0.0 if softcap is None else softcap
        self.tune = tune
        self.init_config(config, tune)

    @property
    def default_config(self) -> dict:
        """``tiles_per_cta`` is the one entry a caller may set: 1 (default) is the kernel with one Q tile per
        CTA (64-key tiles, 192 threads, two CTAs per SM; every head dim); 2 asks for the kernel with two Q
        tiles per CTA (head dim 128: 128-key tiles, 384 threads, persistent grid), which measured slower on
        B200 and is kept as a tuning variant.  The other entries describe the default kernel."""
        return {"block_M": 128, "block_N": 64, "threads": 192, "tiles_per_cta": 1}

    def forward(self, q, k, v, cu_seqlens_q=None, cu_seqlens_kv=None, q_scale=None, k_scale=None,
                v_scale=None, return_lse: bool = False):
        """q ``[B*Sq,H,D]``, k/v ``[B*Skv,Hkv,D]`` of a uniform batch -> o ``[B*Sq,H,D]``."""
        self._require_cuda(q=q, k=k, v=v)
        B, Sq, Skv = self.batch, self.max_seqlen_q, self.max_seqlen_kv
        if q.shape[0] != B * Sq or k.shape[0] != B * Skv:
            raise ValueError(
                f"packed q/k must hold {B}x{Sq} and {B}x{Skv} tokens, got {q.shape[0]} and {k.shape[0]}")
        out = F.gqa_prefill(q.view(B, Sq, self.heads, self.dim), k.view(B, Skv, self.heads_kv, self.dim),
                            v.view(B, Skv, self.heads_kv, self.dim), is_causal=self.is_causal,
                            sm_scale=self.sm_scale, softcap=self.softcap, return_lse=return_lse,
                            window_size_left=self.window_size_left, window_size_right=self.window_size_right,
                            config=self.config)
        if return_lse:
            return out[0].view(q.shape), out[1]
        return out.view(q.shape)


def varlen_prefill_region(call) -> bool:
    """Non-FP8, non-windowed packed prefill that is ragged or asked for as 'varlen'."""
    from .call_spec import uses_sliding_window
    if call.is_fp8 or uses_sliding_window(call):
        return False
    return call.backend == "varlen" or (call.backend == "auto" and not call.is_uniform)


class GQAPrefillVarlenSm100Kernel(Kernel):
    """Ragged packed prefill in the ``gqa_prefill_varlen_fwd_kernel`` slot.

    Replaces the reference's ``GQAPrefillVarlenFwdKernel``
    (``src/tileops/kernels/attention/gqa_prefill_varlen_fwd.py``): per request, keys
    ``cu_seqlens_kv[b] .. cu_seqlens_kv[b+1]`` with a bottom-right aligned causal mask.  Runs the
    tcgen05 prefill kernel in its packed mode (``tb200_gqa_prefill_paged`` without a cache).
    """

    supported_archs = [100]
    general = True

    @classmethod
    def applies(cls, call) -> bool:
        return varlen_prefill_region(call) and call.dim in _PREFILL_DIMS and call.dtype in ATTENTION_DTYPES

    def __init__(self, batch, heads, heads_kv, max_seqlen_q, max_seqlen_kv, dim, is_causal, dtype,
                 sm_scale=None, softcap=0.0, window_size_left=-1, window_size_right=-1,
                 accum_dtype=torch.float32, config: Optional[dict] = None, tune: bool = False,
                 device_index=None) -> None:
        super().__init__(device_index=device_index)
        if dim not in _PREFILL_DIMS:
            raise ValueError(f"{type(self).__name__} supports head dim 64, 128 and 256, got {dim}")
        self.window_size_left, self.window_size_right = window_size_left, window_size_right
        self.batch, self.heads, self.heads_kv, self.dim = batch, heads, heads_kv, dim
        self.max_seqlen_q, self.max_seqlen_kv = max_seqlen_q, max_seqlen_kv
        self.is_causal, self.dtype = is_causal, dtype
        self.sm_scale = dim ** -0.5 if sm_scale is None else sm_scale
        self.softcap = 0.0 if softcap is None else softcap
        self.tune = tune
        self.init_config(config, tune)

    @property
    def default_config(self) -> dict:
        return {"block_M": 128, "block_N": 64, "threads": 192}

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_kv, q_scale=None, k_scale=None, v_scale=None,
                return_lse: bool = False):
        """q ``[total_q,H,D]``, k/v ``[total_kv,Hkv,D]`` -> o ``[total_q,H,D]`` (+ LSE ``[H,total_q]``)."""
        self._require_cuda(q=q, k=k, v=v, cu_seqlens_q=cu_seqlens_q, cu_seqlens_kv=cu_seqlens_kv)
        return F.gqa_prefill_paged(q, k, v, None, None, cu_seqlens_q, None, None, self.max_seqlen_q,
                                   is_causal=self.is_causal, sm_scale=self.sm_scale, softcap=self.softcap,
                                   return_lse=return_lse, cu_seqlens_kv=cu_seqlens_kv,
                                   window_size_left=self.window_size_left,
                                   window_size_right=self.window_size_right)


class GQASlidingWindowVarlenSm100Kernel(GQAPrefillVarlenSm100Kernel):
    """Packed prefill with a sliding window, in the ``gqa_sliding_window_varlen_fwd_kernel`` slot
    (the reference's ``GQASlidingWindowVarlenFwdWgmmaPipelinedKernel``, a Hopper WGMMA kernel).
    Same tcgen05 kernel: key tiles outside the window of a whole 128-row tile are skipped, the
    window edges are masked in registers."""

    @classmethod
    def applies(cls, call) -> bool:
        from .call_spec import uses_sliding_window
        return (uses_sliding_window(call) and not call.is_fp8 and call.backend in ("auto", "sliding_window")
                and call.dim in _PREFILL_DIMS and call.dtype in ATTENTION_DTYPES)


class GQASlidingWindowSm100Kernel(Kernel):
    """Fixed-length (BSHD, Sq == Skv) prefill with a sliding window, in the
    ``gqa_sliding_window_fwd_kernel`` slot (the reference's
    ``GQASlidingWindowFwdWgmmaPipelinedKernel``; constructor keywords as in
    ``src/tileops/ops/attention/gqa.py:1511-1529``)."""

    supported_archs = [100]
    general = True

    @classmethod
    def applies(cls, call) -> bool:
        return call.dim in _PREFILL_DIMS and call.dtype in ATTENTION_DTYPES

    def __init__(self, batch, heads, heads_kv, seq_len, dim, is_causal, window_size_left, window_size_right,
                 dtype, config: Optional[dict] = None, tune: bool = False, device_index=None) -> None:
        super().__init__(device_index=device_index)
        if dim not in _PREFILL_DIMS:
            raise ValueError(f"GQASlidingWindowSm100Kernel supports head dim 64, 128 and 256, got {dim}")
        self.batch, self.heads, self.heads_kv, self.seq_len, self.dim = batch, heads, heads_kv, seq_len, dim
        self.is_causal, self.dtype = is_causal, dtype
        self.window_size_left, self.window_size_right = window_size_left, window_size_right
        self.init_config(config, tune)

    @property
    def default_config(self) -> dict:
        return {"block_M": 128, "block_N": 64, "threads": 192, "tiles_per_cta": 1}

    def forward(self, q, k, v):
        self._require_cuda(q=q, k=k, v=v)
        return F.gqa_prefill(q, k, v, is_causal=self.is_causal, window_size_left=self.window_size_left,
                             window_size_right=self.window_size_right, config=self.config)


class GQAPrefillPagedSm100Kernel(Kernel):
    """Packed prefill over a paged cache with in-place append, in the
    ``gqa_prefill_paged_with_kv_cache_fwd_kernel`` slot.

    Replaces the reference's ``GQAPrefillPagedWithKVCacheFwdKernel``
    (``src/tileops/kernels/attention/gqa_fwd.py:600-1002``); same keyword constructor and
    positional ``forward`` (``src/tileops/ops/attention/gqa.py:866-893,1100-1140``).  The cache has
    the element type of q (the FP8-cache and fused-RoPE slots are not served), so ``k_scale`` /
    ``v_scale`` are accepted and unused, as in the reference's same-type kernel.
    """

    supported_archs = [100]
    general = True

    @classmethod
    def applies(cls, call) -> bool:
        return (call.dtype in ATTENTION_DTYPES and call.dim in _PREFILL_DIMS and not call.fuse_rope
                and call.cache_dtype in (None, call.dtype) and call.page_size >= 16)

    def __init__(self, batch, heads, heads_kv, max_pages_per_req, page_size, dim, is_causal, dtype,
                 sm_scale=None, softcap=0.0, max_position=None, rotary_dim=None,
                 config: Optional[dict] = None, tune: bool = False, device_index=None) -> None:
        super().__init__(device_index=device_index)
        if dim not in _PREFILL_DIMS:
            raise ValueError(f"GQAPrefillPagedSm100Kernel supports head dim 64, 128 and 256, got {dim}")
        if page_size < 16 or page_size & (page_size - 1):
            raise ValueError(f"GQAPrefillPagedSm100Kernel supports power-of-two pages >= 16, got {page_size}")
        self.batch, self.heads, self.heads_kv, self.dim = batch, heads, heads_kv, dim
        self.max_pages_per_req, self.page_size = max_pages_per_req, page_size
        self.is_causal, self.dtype = is_causal, dtype
        self.sm_scale = dim ** -0.5 if sm_scale is None else sm_scale
        self.softcap = 0.0 if softcap is None else softcap
        self.tune = tune
        self.init_config(config, tune)

    @property
    def default_config(self) -> dict:
        return {"block_M": 128, "block_N": 64, "threads": 192}

    def forward(self, q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q, cache_seqlens,
                block_table, max_seqlen_q, cos_table=None, sin_table=None):
        self._require_cuda(q=q, k_new=k_new, v_new=v_new, k_pages=k_pages, v_pages=v_pages)
        if cos_table is not None or sin_table is not None:
            raise ValueError("GQAPrefillPagedSm100Kernel does not fuse RoPE")
        return F.gqa_prefill_paged(q, k_new, v_new, k_pages, v_pages, cu_seqlens_q, cache_seqlens,
                                   block_table, int(max_seqlen_q), page_size=self.page_size,
                                   is_causal=self.is_causal, sm_scale=self.sm_scale, softcap=self.softcap)


class GQAPrefillPagedRopeSm100Kernel(GQAPrefillPagedSm100Kernel):
    """Paged prefill with RoPE, in the ``gqa_prefill_paged_with_kv_cache_rope_fwd_kernel`` slot
    (the reference's ``GQAPrefillPagedWithKVCacheRopeFwdKernel``,
    ``src/tileops/kernels/attention/gqa_fwd.py:1463-2122``).  q and k_new are rotated (GPT-NeoX, at
    positions ``cache_seqlens[b] + i``) by a pass of their own (``tb200_rope_neox_packed``), then the
    paged prefill runs on the rotated tensors, so the pages receive the rotated keys as in the
    reference.  The rotation is not fused into the tcgen05 kernel: q and k_new of a chunk are small next
    to the cached K/V the attention reads."""

    @classmethod
    def applies(cls, call) -> bool:
        return (call.dtype in ATTENTION_DTYPES and call.dim in _PREFILL_DIMS and call.fuse_rope
                and call.cache_dtype in (None, call.dtype) and call.page_size >= 16)

    def __init__(self, batch, heads, heads_kv, max_pages_per_req, page_size, dim, is_causal, dtype,
                 sm_scale=None, softcap=0.0, max_position=None, rotary_dim=None,
                 config: Optional[dict] = None, tune: bool = False, device_index=None) -> None:
        super().__init__(batch, heads, heads_kv, max_pages_per_req, page_size, dim, is_causal, dtype,
                         sm_scale=sm_scale, softcap=softcap, config=config, tune=tune, device_index=device_index)
        if max_position is None:
            raise ValueError("GQAPrefillPagedRopeSm100Kernel needs max_position")
        self.max_position = max_position
        self.rotary_dim = dim if rotary_dim is None else rotary_dim

    def forward(self, q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q, cache_seqlens,
                block_table, max_seqlen_q, cos_table=None, sin_table=None):
        self._require_cuda(q=q, k_new=k_new, v_new=v_new, k_pages=k_pages, v_pages=v_pages)
        if cos_table is None or sin_table is None:
            raise ValueError("GQAPrefillPagedRopeSm100Kernel needs the cos / sin tables")
        q_rot = F.rope_neox_packed(q, cos_table, sin_table, cu_seqlens_q, cache_seqlens, self.rotary_dim)
        k_rot = F.rope_neox_packed(k_new, cos_table, sin_table, cu_seqlens_q, cache_seqlens, self.rotary_dim)
        return F.gqa_prefill_paged(q_rot, k_rot, v_new, k_pages, v_pages, cu_seqlens_q, cache_seqlens,
                                   block_table, int(max_seqlen_q), page_size=self.page_size,
                                   is_causal=self.is_causal, sm_scale=self.sm_scale, softcap=self.softcap)


class GQAPrefillPagedFp8CacheSm100Kernel(GQAPrefillPagedSm100Kernel):
    """Paged prefill over an FP8-e4m3 cache with scalar scales, in the
    ``gqa_prefill_paged_with_fp8_kv_cache_fwd_kernel`` slot (the reference's
    ``GQAPrefillPagedWithFP8KVCacheFwdKernel``, ``src/tileops/kernels/attention/gqa_fwd.py:1005-1460``).
    Default: cached tokens are dequantised into a packed 16-bit K/V (``tb200_fp8_cache_gather``), the packed
    tcgen05 prefill runs on it, and the chunk is quantised into the pages (``tb200_fp8_cache_append``): the
    reference's dequantise-then-attend semantics as three launches.  ``config={"fused": True}`` (head dim 128)
    asks for the one-launch variant that reads the e4m3 pages inside the prefill kernel
    (``tb200_gqa_prefill_paged_e4m3_cache``): no packed copy of the cache, measured 20-30 % slower on B200."""

    @property
    def default_config(self) -> dict:
        return {"block_M": 128, "block_N": 64, "threads": 192, "fused": False}

    @classmethod
    def applies(cls, call) -> bool:
        from .call_spec import fp8_dtype
        return (call.dtype in ATTENTION_DTYPES and call.dim in _PREFILL_DIMS and not call.fuse_rope
                and call.cache_dtype is not None and call.cache_dtype == fp8_dtype())

    def forward(self, q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q, cache_seqlens,
                block_table, max_seqlen_q, cos_table=None, sin_table=None):
        self._require_cuda(q=q, k_new=k_new, v_new=v_new, k_pages=k_pages, v_pages=v_pages)
        if cos_table is not None or sin_table is not None:
            raise ValueError("GQAPrefillPagedFp8CacheSm100Kernel does not apply RoPE")
        return F.gqa_prefill_paged_fp8_cache(q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q,
                                             cache_seqlens, block_table, int(max_seqlen_q),
                                             page_size=self.page_size, is_causal=self.is_causal,
                                             sm_scale=self.sm_scale, softcap=self.softcap,
                                             fused=bool((self.config or {}).get("fused", False)) and self.dim == 128)
