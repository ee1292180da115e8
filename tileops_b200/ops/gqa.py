"""GQA forward operators (L2): the user-facing classes of the path.

Same class names, constructor parameters, ``forward`` signatures, validation order and error
messages as the reference's ``tileops.ops`` GQA ops
(``src/tileops/ops/attention/gqa.py:131-249`` FwdOp, ``:252-552`` PrefillFwdOp, ``:1260-1354``
DecodeWithKVCacheFwdOp, ``:1357-1454`` DecodePagedWithKVCacheFwdOp), so that code written
against the reference runs unchanged; only the kernels behind the ``kernel_map`` slots differ
(hand-written sm_100a CUDA instead of TileLang).  Differences a caller can observe:

* the decode op does not copy K/V to pad them up to ``seqlen_kv`` (the reference ``F.pad``s,
  ``gqa.py:1343-1350``): the live length is a kernel argument;
* the paged decode op performs no host synchronisation per call;
* prefill ops take ``return_lse=True`` to also return the log2-domain LSE ``[B, H, Sq]`` that
  the reference kernels compute and drop (``kernels/attention/gqa_fwd.py:573``);
* ``GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp`` is an addition (FP8-e4m3 cache with one
  fp32 scale per (page, KV head)).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels import (
    GQADecodePagedFp8Sm100Kernel,
    GQADecodePagedSm100Kernel,
    GQADecodeSm100Kernel,
    GQAPrefillSm100Kernel,
)
from ..kernels.kernel_base import Kernel
from .op_base import Op
from .selection import (
    DECODE_KEYS,
    DENSE_PREFILL_KEYS,
    PACKED_PREFILL_KEYS,
    PAGED_DECODE_FP8_KEYS,
    PAGED_DECODE_KEYS,
    AttentionCall,
    check_packed_prefill_request,
    fp8_dtype,
)

__all__ = [
    "GroupedQueryAttentionFwdOp",
    "GroupedQueryAttentionPrefillFwdOp",
    "GroupedQueryAttentionDecodeWithKVCacheFwdOp",
    "GroupedQueryAttentionDecodePagedWithKVCacheFwdOp",
    "GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp",
]


def _validate_attention_dtype(dtype: torch.dtype) -> None:
    if dtype not in (torch.float16, torch.bfloat16):
        raise ValueError(f"Expected dtype torch.float16 or torch.bfloat16, got {dtype}")


def _validate_positive(**values: int) -> None:
    for name, value in values.items():
        if value <= 0:
            raise ValueError(f"{name} must be positive")


def _validate_gqa_dims(heads: int, heads_kv: int, dim: int) -> None:
    _validate_positive(heads=heads, heads_kv=heads_kv)
    if heads % heads_kv != 0:
        raise ValueError("heads must be divisible by heads_kv")
    _validate_positive(dim=dim)


def _attention_scale(dim: int, sm_scale: Optional[float]) -> float:
    return dim ** -0.5 if sm_scale is None else sm_scale


def _score_softcap(softcap: Optional[float]) -> float:
    if softcap is None:
        return 0.0
    if softcap < 0:
        raise ValueError("softcap must be non-negative")
    return softcap


def _build_packed_prefill_kernel(kernel_map: Dict[str, type], key: str, call: AttentionCall) -> Kernel:
    # every implementation of the slot takes this keyword constructor (reference gqa.py:113-128)
    return kernel_map[key](
        batch=call.batch, heads=call.heads, heads_kv=call.heads_kv,
        max_seqlen_q=call.max_seqlen_q, max_seqlen_kv=call.max_seqlen_kv, dim=call.dim,
        is_causal=call.is_causal, dtype=call.dtype, sm_scale=call.sm_scale, softcap=call.softcap,
        window_size_left=call.window_size_left, window_size_right=call.window_size_right,
        accum_dtype=call.accum_dtype, tune=call.tune)


def _run_prefill_kernel(kernel, args, return_lse: bool):
    if return_lse:
        return kernel(*args, return_lse=True)
    return kernel(*args)


class GroupedQueryAttentionFwdOp(Op):
    """Square (Sq == Skv) GQA forward. Layout: BSHD."""

    def __init__(self, batch: int, heads: int, heads_kv: int, seq_len: int, dim: int,
                 is_causal: bool = True, sm_scale: Optional[float] = None,
                 softcap: Optional[float] = None, kernel_map: Optional[Dict[str, type]] = None,
                 tune: bool = False) -> None:
        _validate_gqa_dims(heads, heads_kv, dim)
        _validate_positive(batch=batch, seq_len=seq_len)
        self.batch, self.heads, self.heads_kv = batch, heads, heads_kv
        self.seq_len, self.dim, self.is_causal = seq_len, dim, is_causal
        self.sm_scale = _attention_scale(dim, sm_scale)
        self.softcap = _score_softcap(softcap)
        self.tune = tune
        self.dispatch_kernel(kernel_map)
        self._cu_seqlens: Dict[torch.device, torch.Tensor] = {}

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_prefill_fwd_kernel": GQAPrefillSm100Kernel}

    def attention_call(self, dtype: torch.dtype) -> AttentionCall:
        return AttentionCall(
            dtype=dtype, batch=self.batch, heads=self.heads, heads_kv=self.heads_kv, dim=self.dim,
            max_seqlen_q=self.seq_len, max_seqlen_kv=self.seq_len, is_causal=self.is_causal,
            sm_scale=self.sm_scale, softcap=self.softcap, backend="dense", is_fp8=False,
            is_uniform=True, tune=self.tune)

    def _get_kernel(self, inputs, dtype: torch.dtype) -> Kernel:
        _validate_attention_dtype(dtype)
        call = self.attention_call(dtype)
        key = self.select_kernel_key(DENSE_PREFILL_KEYS, call)
        return self.get_or_build_kernel(
            key, inputs, key=dtype, build=lambda: _build_packed_prefill_kernel(self.kernel_map, key, call))

    def _uniform_cu_seqlens(self, device: torch.device) -> torch.Tensor:
        cu = self._cu_seqlens.get(device)
        if cu is None:
            cu = torch.arange(self.batch + 1, device=device, dtype=torch.int32) * self.seq_len
            self._cu_seqlens[device] = cu
        return cu

    def _infer_output_shapes(self, q_shape, k_shape, v_shape) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, return_lse: bool = False):
        expected_q = (self.batch, self.seq_len, self.heads, self.dim)
        expected_kv = (self.batch, self.seq_len, self.heads_kv, self.dim)
        if tuple(q.shape) != expected_q:
            raise ValueError(f"q must have shape {expected_q}, got {tuple(q.shape)}")
        if tuple(k.shape) != expected_kv:
            raise ValueError(f"k must have shape {expected_kv}, got {tuple(k.shape)}")
        if tuple(v.shape) != expected_kv:
            raise ValueError(f"v must have shape {expected_kv}, got {tuple(v.shape)}")
        self._validate_dtypes(q, k, v)
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        self.dtype = q.dtype
        cu = self._uniform_cu_seqlens(q.device)
        args = (q.view(-1, self.heads, self.dim), k.view(-1, self.heads_kv, self.dim),
                v.view(-1, self.heads_kv, self.dim), cu, cu)
        out = _run_prefill_kernel(self._get_kernel((q, k, v), q.dtype), args, return_lse)
        if return_lse:
            return out[0].view(q.shape), out[1]
        return out.view(q.shape)


class GroupedQueryAttentionPrefillFwdOp(Op):
    """Canonical packed (THD) GQA prefill; dense requests carry uniform ``cu_seqlens``.

    ``dtype`` is the element type of ``o``; for fp16/bf16 inputs it must equal theirs.
    """

    def __init__(self, batch: int, heads: int, heads_kv: int, dim: int, max_seqlen_q: int,
                 max_seqlen_kv: int, dtype: torch.dtype = torch.float16, is_causal: bool = True,
                 sm_scale: Optional[float] = None, softcap: Optional[float] = None,
                 window_size_left: int = -1, window_size_right: int = -1, backend: str = "auto",
                 validate_uniform_cu_seqlens: bool = True,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        _validate_gqa_dims(heads, heads_kv, dim)
        _validate_positive(batch=batch, max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv)
        if is_causal and max_seqlen_q > max_seqlen_kv:
            raise ValueError("causal prefill requires max_seqlen_q <= max_seqlen_kv")
        if window_size_left != -1 and window_size_left < 0:
            raise ValueError(f"window_size_left must be -1 (unlimited) or >= 0, got {window_size_left}")
        if window_size_right != -1 and window_size_right < 0:
            raise ValueError(f"window_size_right must be -1 (unlimited) or >= 0, got {window_size_right}")
        if backend not in ("auto", "dense", "varlen", "fp8", "sliding_window"):
            raise ValueError("backend must be one of 'auto', 'dense', 'varlen', 'fp8', or 'sliding_window'")
        if backend == "auto" and not validate_uniform_cu_seqlens:
            raise ValueError("backend='auto' requires validate_uniform_cu_seqlens=True.")
        _validate_attention_dtype(dtype)
        self.batch, self.heads, self.heads_kv, self.dim = batch, heads, heads_kv, dim
        self.max_seqlen_q, self.max_seqlen_kv = max_seqlen_q, max_seqlen_kv
        self.dtype, self.is_causal = dtype, is_causal
        self.sm_scale = _attention_scale(dim, sm_scale)
        self.softcap = _score_softcap(softcap)
        self.window_size_left, self.window_size_right = window_size_left, window_size_right
        self.backend = backend
        self.validate_uniform_cu_seqlens = validate_uniform_cu_seqlens
        self.tune = tune
        self._roofline_kwargs = None
        self._uniform_cu_cache: dict = {}
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_prefill_fwd_kernel": GQAPrefillSm100Kernel}

    def attention_call(self, *, is_fp8: bool, is_uniform: bool) -> AttentionCall:
        return AttentionCall(
            dtype=self.dtype, batch=self.batch, heads=self.heads, heads_kv=self.heads_kv, dim=self.dim,
            max_seqlen_q=self.max_seqlen_q, max_seqlen_kv=self.max_seqlen_kv, is_causal=self.is_causal,
            sm_scale=self.sm_scale, softcap=self.softcap, window_size_left=self.window_size_left,
            window_size_right=self.window_size_right, backend=self.backend, is_fp8=is_fp8,
            is_uniform=is_uniform, tune=self.tune)

    def _infer_output_shapes(self, q_shape, k_shape, v_shape, cu_seqlens_q_shape, cu_seqlens_kv_shape,
                             q_scale_shape, k_scale_shape, v_scale_shape) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def _validate_dtypes(self, q, k, v, cu_seqlens_q, cu_seqlens_kv, q_scale, k_scale, v_scale) -> None:
        f8 = fp8_dtype()
        if f8 is not None and q.dtype == f8:
            if k.dtype != f8 or v.dtype != f8:
                raise ValueError("FP8 prefill requires q/k/v to all be torch.float8_e4m3fn.")
        elif q.dtype != self.dtype or k.dtype != self.dtype or v.dtype != self.dtype:
            raise ValueError(f"q/k/v dtype must match op dtype {self.dtype}.")
        if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_kv.dtype != torch.int32:
            raise ValueError("cu_seqlens_q/cu_seqlens_kv must be torch.int32.")
        if any(s.dtype != torch.float32 for s in (q_scale, k_scale, v_scale)):
            raise ValueError("q_scale/k_scale/v_scale must be torch.float32.")

    def _validate_common_shapes(self, q, k, v, cu_seqlens_q, cu_seqlens_kv, q_scale, k_scale, v_scale) -> None:
        named = (("q", q), ("k", k), ("v", v), ("cu_seqlens_q", cu_seqlens_q),
                 ("cu_seqlens_kv", cu_seqlens_kv), ("q_scale", q_scale), ("k_scale", k_scale),
                 ("v_scale", v_scale))
        for name, t in named:
            if t.device.type != "cuda":
                raise ValueError(f"{name} must be on a cuda device, got {t.device}")
            if not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        if q.ndim != 3 or tuple(q.shape[1:]) != (self.heads, self.dim):
            raise ValueError(f"q must have shape [T, {self.heads}, {self.dim}], got {tuple(q.shape)}")
        for name, t in (("k", k), ("v", v)):
            if t.ndim != 3 or tuple(t.shape[1:]) != (self.heads_kv, self.dim):
                raise ValueError(f"{name} must have shape [T, {self.heads_kv}, {self.dim}], got {tuple(t.shape)}")
        if v.shape[0] != k.shape[0]:
            raise ValueError(f"v.shape[0] ({v.shape[0]}) must equal k.shape[0] ({k.shape[0]})")
        cu_shape = (self.batch + 1,)
        for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_kv", cu_seqlens_kv)):
            if tuple(t.shape) != cu_shape:
                raise ValueError(f"{name} must have shape {cu_shape}, got {tuple(t.shape)}")
        scale_shape = (self.batch, self.heads_kv)
        for name, t in (("q_scale", q_scale), ("k_scale", k_scale), ("v_scale", v_scale)):
            if tuple(t.shape) != scale_shape:
                raise ValueError(f"{name} must have shape {scale_shape}, got {tuple(t.shape)}")

    def _uniform_cu_seqlens(self, cu_seqlens: torch.Tensor, seq_len: int) -> bool:
        key = (seq_len, cu_seqlens.device, cu_seqlens.dtype)
        expected = self._uniform_cu_cache.get(key)
        if expected is None:
            expected = torch.arange(self.batch + 1, device=cu_seqlens.device, dtype=cu_seqlens.dtype) * seq_len
            self._uniform_cu_cache[key] = expected
        return bool(torch.equal(cu_seqlens, expected))  # device->host sync, as in the reference

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_kv, q_scale, k_scale, v_scale,
                return_lse: bool = False):
        self._validate_dtypes(q, k, v, cu_seqlens_q, cu_seqlens_kv, q_scale, k_scale, v_scale)
        self._validate_common_shapes(q, k, v, cu_seqlens_q, cu_seqlens_kv, q_scale, k_scale, v_scale)
        if self.backend == "auto" or (self.backend in ("dense", "fp8") and self.validate_uniform_cu_seqlens):
            is_uniform = (self._uniform_cu_seqlens(cu_seqlens_q, self.max_seqlen_q)
                          and self._uniform_cu_seqlens(cu_seqlens_kv, self.max_seqlen_kv))
        else:
            is_uniform = True
        f8 = fp8_dtype()
        call = self.attention_call(is_fp8=f8 is not None and q.dtype == f8, is_uniform=is_uniform)
        check_packed_prefill_request(call)
        key = self.select_kernel_key(PACKED_PREFILL_KEYS, call)
        inputs = (q, k, v, cu_seqlens_q, cu_seqlens_kv, q_scale, k_scale, v_scale)
        kernel = self.get_or_build_kernel(
            key, inputs, key=call.dtype, build=lambda: _build_packed_prefill_kernel(self.kernel_map, key, call))
        out = _run_prefill_kernel(kernel, inputs, return_lse)
        self._roofline_kwargs = {
            "q_shape": tuple(q.shape), "k_shape": tuple(k.shape), "batch": self.batch,
            "max_seqlen_q": self.max_seqlen_q, "max_seqlen_kv": self.max_seqlen_kv,
            "cu_seqlens_q": cu_seqlens_q, "cu_seqlens_kv": cu_seqlens_kv,
            "is_causal": self.is_causal, "dtype": q.dtype}
        return out

    def eval_roofline(self) -> tuple:
        if self._roofline_kwargs is None:
            raise RuntimeError(f"{type(self).__name__}.eval_roofline() requires a prior forward() call")
        from ..perf.formulas import gqa_prefill_varlen_fwd_roofline
        return gqa_prefill_varlen_fwd_roofline(**self._roofline_kwargs)


class GroupedQueryAttentionDecodeWithKVCacheFwdOp(Op):
    """Single-token decode over a contiguous cache. Layout: q BHD, k/v BSHD."""

    def __init__(self, batch: int, heads: int, heads_kv: int, seqlen_kv: int, dim: int,
                 sm_scale: Optional[float] = None, softcap: Optional[float] = None,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        _validate_gqa_dims(heads, heads_kv, dim)
        self.batch, self.heads, self.heads_kv = batch, heads, heads_kv
        self.seqlen_kv, self.dim = seqlen_kv, dim
        self.sm_scale = _attention_scale(dim, sm_scale)
        self.softcap = _score_softcap(softcap)
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_decode_kernel": GQADecodeSm100Kernel}

    def attention_call(self, dtype: torch.dtype) -> AttentionCall:
        return AttentionCall(dtype=dtype, batch=self.batch, heads=self.heads, heads_kv=self.heads_kv,
                             seqlen_kv=self.seqlen_kv, dim=self.dim, sm_scale=self.sm_scale,
                             softcap=self.softcap, tune=self.tune)

    def _get_kernel(self, inputs, dtype: torch.dtype) -> Kernel:
        _validate_attention_dtype(dtype)
        call = self.attention_call(dtype)
        key = self.select_kernel_key(DECODE_KEYS, call)
        return self.get_or_build_kernel(key, inputs, key=dtype, build=lambda: self.kernel_map[key](
            call.batch, call.heads, call.heads_kv, call.seqlen_kv, call.dim, call.dtype,
            sm_scale=call.sm_scale, softcap=call.softcap, tune=call.tune))

    def _infer_output_shapes(self, q_shape, k_shape, v_shape) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        real_seqlen_kv = k.shape[1]
        if real_seqlen_kv > self.seqlen_kv:
            raise ValueError(f"k holds {real_seqlen_kv} tokens, more than seqlen_kv={self.seqlen_kv}")
        self._validate_dtypes(q, k, v)
        self.dtype = q.dtype
        return self._get_kernel((q, k, v), q.dtype)(q, k, v, real_seqlen_kv)


class GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(Op):
    """Single-token decode over a paged cache. q ``[B,H,D]``; k, v physical pool
    ``[seqlen_kv, heads_kv, dim]``; real_seqlen_kv ``[B]`` int32; block_table ``[B, num_pages]`` int32."""

    _KEYS = PAGED_DECODE_KEYS

    def __init__(self, batch: int, heads: int, heads_kv: int, seqlen_kv: int, dim: int, page_size: int,
                 sm_scale: Optional[float] = None, softcap: Optional[float] = None,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        _validate_gqa_dims(heads, heads_kv, dim)
        self.batch, self.heads, self.heads_kv = batch, heads, heads_kv
        self.seqlen_kv, self.dim, self.page_size = seqlen_kv, dim, page_size
        _validate_positive(page_size=page_size)
        self.sm_scale = _attention_scale(dim, sm_scale)
        self.softcap = _score_softcap(softcap)
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_decode_paged_kernel": GQADecodePagedSm100Kernel}

    def attention_call(self, dtype: torch.dtype) -> AttentionCall:
        return AttentionCall(dtype=dtype, batch=self.batch, heads=self.heads, heads_kv=self.heads_kv,
                             seqlen_kv=self.seqlen_kv, dim=self.dim, page_size=self.page_size,
                             sm_scale=self.sm_scale, softcap=self.softcap, tune=self.tune)

    def _get_kernel(self, inputs, dtype: torch.dtype) -> Kernel:
        _validate_attention_dtype(dtype)
        call = self.attention_call(dtype)
        key = self.select_kernel_key(self._KEYS, call)
        return self.get_or_build_kernel(key, inputs, key=dtype, build=lambda: self.kernel_map[key](
            call.batch, call.heads, call.heads_kv, call.seqlen_kv, call.dim, call.page_size, call.dtype,
            sm_scale=call.sm_scale, softcap=call.softcap, tune=call.tune))

    def _infer_output_shapes(self, q_shape, k_shape, v_shape, real_seqlen_kv_shape,
                             block_table_shape) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q, k, v, real_seqlen_kv, block_table) -> torch.Tensor:
        self.dtype = q.dtype
        return self._get_kernel((q, k, v, real_seqlen_kv, block_table), q.dtype)(
            q, k, v, real_seqlen_kv, block_table)


class GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp(GroupedQueryAttentionDecodePagedWithKVCacheFwdOp):
    """Paged decode over an FP8-e4m3 cache: ``forward(q, k_fp8, v_fp8, k_scale, v_scale,
    real_seqlen_kv, block_table)`` with fp32 scales ``[seqlen_kv / page_size, heads_kv]``
    (``x = float(x_fp8) * scale``).  Matches dequantise-then-attend."""

    _KEYS = PAGED_DECODE_FP8_KEYS

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_decode_paged_fp8_kernel": GQADecodePagedFp8Sm100Kernel}

    def _infer_output_shapes(self, q_shape, *rest) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q, k, v, k_scale, v_scale, real_seqlen_kv, block_table) -> torch.Tensor:
        self._validate_dtypes(q, k, v, k_scale, v_scale, real_seqlen_kv, block_table)
        expected = (self.seqlen_kv // self.page_size, self.heads_kv)
        for name, t in (("k_scale", k_scale), ("v_scale", v_scale)):
            if tuple(t.shape) != expected:
                raise ValueError(f"{name} must have shape {expected}, got {tuple(t.shape)}")
        self.dtype = q.dtype
        self.cache_dtype = k.dtype
        return self._get_kernel((q, k, v, k_scale, v_scale, real_seqlen_kv, block_table), q.dtype)(
            q, k, v, k_scale, v_scale, real_seqlen_kv, block_table)

    def eval_roofline(self) -> tuple:
        from ..perf.formulas import gqa_decode_paged_roofline
        data = dict(vars(self))
        data["dtype"] = getattr(self, "cache_dtype", None) or fp8_dtype()
        return gqa_decode_paged_roofline(data)
