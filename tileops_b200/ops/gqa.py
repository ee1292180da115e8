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
    GQAPrefillPagedFp8CacheSm100Kernel,
    GQAPrefillPagedRopeSm100Kernel,
    GQAPrefillPagedSm100Kernel,
    GQAPrefillSm100Kernel,
    GQAPrefillVarlenSm100Kernel,
    GQASlidingWindowSm100Kernel,
    GQASlidingWindowVarlenSm100Kernel,
)
from ..kernels.kernel_base import Kernel
from .op_base import Op
from .selection import (
    DECODE_KEYS,
    DENSE_PREFILL_KEYS,
    PACKED_PREFILL_KEYS,
    PAGED_DECODE_FP8_KEYS,
    PAGED_DECODE_KEYS,
    PAGED_PREFILL_KEYS,
    AttentionCall,
    check_packed_prefill_request,
    fp8_dtype,
)

__all__ = [
    "GroupedQueryAttentionFwdOp",
    "GroupedQueryAttentionPrefillFwdOp",
    "GroupedQueryAttentionPrefillVarlenFwdOp",
    "GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp",
    "GroupedQueryAttentionSlidingWindowFwdOp",
    "GroupedQueryAttentionSlidingWindowVarlenFwdOp",
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
        return {"gqa_prefill_fwd_kernel": GQAPrefillSm100Kernel,
                "gqa_prefill_varlen_fwd_kernel": GQAPrefillVarlenSm100Kernel,
                "gqa_sliding_window_varlen_fwd_kernel": GQASlidingWindowVarlenSm100Kernel}

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


class GroupedQueryAttentionPrefillVarlenFwdOp(Op):
    """Packed variable-length GQA prefill (THD).  Request b owns rows ``cu_seqlens_q[b]:cu_seqlens_q[b+1]``
    of q and ``cu_seqlens_kv[b]:cu_seqlens_kv[b+1]`` of k/v; the causal mask is bottom-right aligned per
    request (key j visible to row i iff ``j <= i + (kv_len - q_len)``).  Mirrors
    ``src/tileops/ops/attention/gqa.py:555-762`` of the reference."""

    def __init__(self, batch: int, heads: int, heads_kv: int, dim: int, max_seqlen_q: int,
                 max_seqlen_kv: int, is_causal: bool = True, sm_scale: Optional[float] = None,
                 softcap: Optional[float] = None, validate_inputs: bool = False,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        _validate_gqa_dims(heads, heads_kv, dim)
        _validate_positive(batch=batch, max_seqlen_q=max_seqlen_q, max_seqlen_kv=max_seqlen_kv)
        self.batch, self.heads, self.heads_kv, self.dim = batch, heads, heads_kv, dim
        self.max_seqlen_q, self.max_seqlen_kv = max_seqlen_q, max_seqlen_kv
        self.is_causal = is_causal
        self.sm_scale = _attention_scale(dim, sm_scale)
        self.softcap = _score_softcap(softcap)
        self.validate_inputs = validate_inputs
        self._roofline_kwargs = None
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_prefill_varlen_fwd_kernel": GQAPrefillVarlenSm100Kernel}

    def _get_kernel(self, inputs, dtype: torch.dtype) -> Kernel:
        _validate_attention_dtype(dtype)
        return self.get_or_build_kernel(
            "gqa_prefill_varlen_fwd_kernel", inputs, key=dtype,
            build=lambda: self.kernel_map["gqa_prefill_varlen_fwd_kernel"](
                batch=self.batch, heads=self.heads, heads_kv=self.heads_kv, max_seqlen_q=self.max_seqlen_q,
                max_seqlen_kv=self.max_seqlen_kv, dim=self.dim, is_causal=self.is_causal, dtype=dtype,
                sm_scale=self.sm_scale, softcap=self.softcap, tune=self.tune))

    @staticmethod
    def _lengths_from_cu_seqlens(cu_seqlens: torch.Tensor) -> list:
        values = [int(x) for x in cu_seqlens.detach().cpu().tolist()]
        return [b - a for a, b in zip(values[:-1], values[1:])]

    def _validate_forward_inputs(self, q, k, v, cu_seqlens_q, cu_seqlens_kv) -> None:
        named = (("q", q), ("k", k), ("v", v), ("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_kv", cu_seqlens_kv))
        for name, t in named:
            if not t.is_cuda:
                raise ValueError(f"{name} must be a CUDA tensor")
            if not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        if q.ndim != 3 or tuple(q.shape[1:]) != (self.heads, self.dim):
            raise ValueError(f"q must have shape [T, {self.heads}, {self.dim}], got {tuple(q.shape)}")
        for name, t in (("k", k), ("v", v)):
            if t.ndim != 3 or tuple(t.shape[1:]) != (self.heads_kv, self.dim):
                raise ValueError(f"{name} must have shape [T, {self.heads_kv}, {self.dim}], got {tuple(t.shape)}")
            if t.dtype != q.dtype:
                raise ValueError(f"Expected {name}.dtype {q.dtype}, got {t.dtype}")
        for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cu_seqlens_kv", cu_seqlens_kv)):
            if tuple(t.shape) != (self.batch + 1,):
                raise ValueError(f"{name} must have shape ({self.batch + 1},), got {tuple(t.shape)}")
            if t.dtype != torch.int32:
                raise ValueError(f"Expected {name}.dtype torch.int32, got {t.dtype}")
        if v.shape[0] != k.shape[0]:
            raise ValueError(f"v.shape[0] ({v.shape[0]}) must equal k.shape[0] ({k.shape[0]})")
        if not self.validate_inputs:
            return
        cu_q = [int(x) for x in cu_seqlens_q.detach().cpu().tolist()]
        cu_kv = [int(x) for x in cu_seqlens_kv.detach().cpu().tolist()]
        if cu_q[0] != 0:
            raise ValueError(f"cu_seqlens_q[0] must be 0, got {cu_q[0]}")
        if cu_kv[0] != 0:
            raise ValueError(f"cu_seqlens_kv[0] must be 0, got {cu_kv[0]}")
        if cu_q[-1] != q.shape[0]:
            raise ValueError(f"cu_seqlens_q[-1] ({cu_q[-1]}) must equal q.shape[0] ({q.shape[0]})")
        if cu_kv[-1] != k.shape[0]:
            raise ValueError(f"cu_seqlens_kv[-1] ({cu_kv[-1]}) must equal k.shape[0] ({k.shape[0]})")
        q_lens = [b - a for a, b in zip(cu_q[:-1], cu_q[1:])]
        kv_lens = [b - a for a, b in zip(cu_kv[:-1], cu_kv[1:])]
        if any(n < 0 for n in q_lens):
            raise ValueError("cu_seqlens_q must be non-decreasing")
        if any(n < 0 for n in kv_lens):
            raise ValueError("cu_seqlens_kv must be non-decreasing")
        for q_len, kv_len in zip(q_lens, kv_lens):
            if q_len <= 0:
                raise ValueError("all q sequence lengths must be positive")
            if kv_len <= 0:
                raise ValueError("all kv sequence lengths must be positive")
            if self.is_causal and q_len > kv_len:
                raise ValueError("causal varlen prefill requires every q_len <= kv_len")
        if self.max_seqlen_q < max(q_lens):
            raise ValueError(f"max_seqlen_q ({self.max_seqlen_q}) must be >= actual max Q "
                             f"sequence length ({max(q_lens)})")
        if self.max_seqlen_kv < max(kv_lens):
            raise ValueError(f"max_seqlen_kv ({self.max_seqlen_kv}) must be >= actual max KV "
                             f"sequence length ({max(kv_lens)})")

    def _infer_output_shapes(self, q_shape, *rest) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_kv) -> torch.Tensor:
        self._validate_forward_inputs(q, k, v, cu_seqlens_q, cu_seqlens_kv)
        self.dtype = q.dtype
        tensors = (q, k, v, cu_seqlens_q, cu_seqlens_kv)
        out = self._get_kernel(tensors, q.dtype)(*tensors)
        self._roofline_kwargs = {
            "q_shape": tuple(q.shape), "k_shape": tuple(k.shape), "batch": self.batch,
            "max_seqlen_q": self.max_seqlen_q, "max_seqlen_kv": self.max_seqlen_kv,
            "cu_seqlens_q": cu_seqlens_q, "cu_seqlens_kv": cu_seqlens_kv,
            "is_causal": self.is_causal, "dtype": self.dtype}
        return out

    def eval_roofline(self) -> tuple:
        if self._roofline_kwargs is None:
            raise RuntimeError(f"{type(self).__name__}.eval_roofline() requires a prior forward() call")
        from ..perf.formulas import gqa_prefill_varlen_fwd_roofline
        kwargs = dict(self._roofline_kwargs)
        kwargs["q_lens"] = self._lengths_from_cu_seqlens(kwargs.pop("cu_seqlens_q"))
        kwargs["kv_lens"] = self._lengths_from_cu_seqlens(kwargs.pop("cu_seqlens_kv"))
        return gqa_prefill_varlen_fwd_roofline(**kwargs)


def _paged_cache_dtype(cache_dtype: Optional[torch.dtype]) -> Optional[torch.dtype]:
    if cache_dtype is None:
        return None
    if cache_dtype != fp8_dtype():
        _validate_attention_dtype(cache_dtype)
    return cache_dtype


class GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp(Op):
    """Packed GQA prefill with paged KV-cache append (THD).

    The chunk is packed by request; ``cache_seqlens`` holds every request's logical KV length
    before the append; ``block_table`` maps logical to physical pages of ``k_pages`` / ``v_pages``,
    which are modified in place.  Mirrors ``src/tileops/ops/attention/gqa.py:765-1157`` of the
    reference (constructor, validation order and messages, positional ``forward``).  Served here:
    a cache of q's element type, head dim 64 / 128, power-of-two pages >= 16, with or without
    ``fuse_rope=True`` (GPT-NeoX rotation of q and k_new at positions ``cache_seqlens[b] + i``; the
    pages receive the rotated keys), or an FP8-e4m3 cache with scalar ``k_scale`` / ``v_scale``
    (``cache_dtype=torch.float8_e4m3fn``: cached tokens dequantised, the chunk quantised on append).
    """

    def __init__(self, batch: int, heads: int, heads_kv: int, max_pages_per_req: int, page_size: int,
                 dim: int, is_causal: bool = True, cache_dtype: Optional[torch.dtype] = None,
                 sm_scale: Optional[float] = None, softcap: Optional[float] = None,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False,
                 fuse_rope: bool = False, rope_base: float = 10000.0, max_position: Optional[int] = None,
                 rotary_dim: Optional[int] = None) -> None:
        _validate_gqa_dims(heads, heads_kv, dim)
        if fuse_rope:
            rotary_dim = dim if rotary_dim is None else rotary_dim
            if rotary_dim <= 0 or rotary_dim > dim or rotary_dim % 2:
                raise ValueError(f"rotary_dim must be an even value in (0, {dim}], got {rotary_dim}")
            if max_position is None:
                raise ValueError("max_position is required when fuse_rope=True")
            _validate_positive(max_position=max_position)
        elif rotary_dim is not None:
            raise ValueError("rotary_dim requires fuse_rope=True")
        _validate_positive(batch=batch, max_pages_per_req=max_pages_per_req, page_size=page_size)
        if page_size & (page_size - 1) != 0:
            raise ValueError("page_size must be a power of two")
        cache_dtype = _paged_cache_dtype(cache_dtype)
        if fuse_rope and cache_dtype is not None and cache_dtype == fp8_dtype():
            raise ValueError("fuse_rope is not supported with FP8 paged KV cache yet")
        self.batch, self.heads, self.heads_kv = batch, heads, heads_kv
        self.groups = heads // heads_kv
        self.max_pages_per_req, self.page_size = max_pages_per_req, page_size
        self.max_cache_len = max_pages_per_req * page_size
        self.dim, self.is_causal = dim, is_causal
        self.cache_dtype = cache_dtype          # None: the cache has forward's element type
        self.sm_scale = _attention_scale(dim, sm_scale)
        self.softcap = _score_softcap(softcap)
        self.fuse_rope, self.rope_base = fuse_rope, rope_base
        self.max_position, self.rotary_dim = max_position, rotary_dim
        self._rope_tables: dict = {}
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_prefill_paged_with_kv_cache_fwd_kernel": GQAPrefillPagedSm100Kernel,
                "gqa_prefill_paged_with_kv_cache_rope_fwd_kernel": GQAPrefillPagedRopeSm100Kernel,
                "gqa_prefill_paged_with_fp8_kv_cache_fwd_kernel": GQAPrefillPagedFp8CacheSm100Kernel}

    def _resolved_cache_dtype(self, dtype: torch.dtype) -> torch.dtype:
        return dtype if self.cache_dtype is None else self.cache_dtype

    def attention_call(self, dtype: torch.dtype) -> AttentionCall:
        return AttentionCall(
            dtype=dtype, batch=self.batch, heads=self.heads, heads_kv=self.heads_kv, dim=self.dim,
            max_pages_per_req=self.max_pages_per_req, page_size=self.page_size, is_causal=self.is_causal,
            sm_scale=self.sm_scale, softcap=self.softcap, cache_dtype=self._resolved_cache_dtype(dtype),
            fuse_rope=self.fuse_rope, max_position=self.max_position, rotary_dim=self.rotary_dim,
            tune=self.tune)

    def _get_kernel(self, inputs, key: str, call: AttentionCall) -> Kernel:
        return self.get_or_build_kernel(key, inputs, key=call.dtype, build=lambda: self.kernel_map[key](
            batch=call.batch, heads=call.heads, heads_kv=call.heads_kv,
            max_pages_per_req=call.max_pages_per_req, page_size=call.page_size, dim=call.dim,
            is_causal=call.is_causal, dtype=call.dtype, sm_scale=call.sm_scale, softcap=call.softcap,
            max_position=call.max_position, rotary_dim=call.rotary_dim, tune=call.tune))

    def _validate_forward_inputs(self, q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q,
                                 cache_seqlens, block_table, max_seqlen_q) -> None:
        named = (("q", q), ("k_new", k_new), ("v_new", v_new), ("k_pages", k_pages), ("v_pages", v_pages),
                 ("k_scale", k_scale), ("v_scale", v_scale), ("cu_seqlens_q", cu_seqlens_q),
                 ("cache_seqlens", cache_seqlens), ("block_table", block_table))
        for name, t in named:
            if t.device.type != "cuda":
                raise ValueError(f"{name} must be on a cuda device, got {t.device}")
            if not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        if q.ndim != 3 or tuple(q.shape[1:]) != (self.heads, self.dim):
            raise ValueError(f"q must have shape [total_q, {self.heads}, {self.dim}], got {q.shape}")
        if k_new.ndim != 3 or tuple(k_new.shape[1:]) != (self.heads_kv, self.dim):
            raise ValueError(f"k_new must have shape [total_q, {self.heads_kv}, {self.dim}], got {k_new.shape}")
        if v_new.shape != k_new.shape:
            raise ValueError(f"v_new must have the same shape as k_new, got {v_new.shape} and {k_new.shape}")
        if k_new.shape[0] != q.shape[0]:
            raise ValueError(f"k_new.shape[0] ({k_new.shape[0]}) must equal q.shape[0] ({q.shape[0]})")
        if k_pages.ndim != 3 or tuple(k_pages.shape[1:]) != (self.heads_kv, self.dim):
            raise ValueError(f"k_pages must have shape [physical_tokens, {self.heads_kv}, {self.dim}], "
                             f"got {k_pages.shape}")
        if v_pages.shape != k_pages.shape:
            raise ValueError(f"v_pages must have the same shape as k_pages, got {v_pages.shape} and "
                             f"{k_pages.shape}")
        if k_pages.shape[0] % self.page_size != 0:
            raise ValueError("k_pages physical token dimension must be divisible by page_size")
        if k_scale.shape != (1,) or v_scale.shape != (1,):
            raise ValueError(f"k_scale and v_scale must have shape (1,), got {k_scale.shape} and {v_scale.shape}")
        if cu_seqlens_q.shape != (self.batch + 1,):
            raise ValueError(f"cu_seqlens_q shape must be ({self.batch + 1},), got {tuple(cu_seqlens_q.shape)}")
        if cache_seqlens.shape != (self.batch,):
            raise ValueError(f"cache_seqlens shape must be ({self.batch},), got {tuple(cache_seqlens.shape)}")
        if block_table.shape != (self.batch, self.max_pages_per_req):
            raise ValueError(f"block_table shape must be ({self.batch}, {self.max_pages_per_req}), "
                             f"got {tuple(block_table.shape)}")
        _validate_attention_dtype(q.dtype)
        cache_dtype = self._resolved_cache_dtype(q.dtype)
        f8 = fp8_dtype()
        if cache_dtype != q.dtype and cache_dtype != f8:
            raise ValueError("cache_dtype must be either same as the q element type or "
                             f"torch.float8_e4m3fn, got {cache_dtype}")
        for name, t in (("k_new", k_new), ("v_new", v_new)):
            if t.dtype != q.dtype:
                raise ValueError(f"Expected {name}.dtype {q.dtype}, got {t.dtype}")
        for name, t in (("k_pages", k_pages), ("v_pages", v_pages)):
            if t.dtype != cache_dtype:
                raise ValueError(f"Expected {name}.dtype {cache_dtype}, got {t.dtype}")
        for name, t in (("k_scale", k_scale), ("v_scale", v_scale)):
            if t.dtype != torch.float32:
                raise ValueError(f"{name} must have dtype torch.float32, got {t.dtype}")
            if cache_dtype == f8 and not torch.all(torch.isfinite(t) & (t > 0)).item():
                raise ValueError(f"{name} must contain finite positive values")
        for name, t in (("cu_seqlens_q", cu_seqlens_q), ("cache_seqlens", cache_seqlens),
                        ("block_table", block_table)):
            if t.dtype != torch.int32:
                raise ValueError(f"{name} must have dtype torch.int32, got {t.dtype}")
        # the range checks below read the tensors on the host, as the reference's do
        if int(cu_seqlens_q[0].item()) != 0:
            raise ValueError("cu_seqlens_q[0] must be 0")
        q_lens = cu_seqlens_q[1:] - cu_seqlens_q[:-1]
        if torch.any(q_lens < 0).item():
            raise ValueError("cu_seqlens_q must be non-decreasing")
        total_q = int(cu_seqlens_q[-1].item())
        if total_q != q.shape[0]:
            raise ValueError(f"cu_seqlens_q[-1] ({total_q}) must equal q.shape[0] ({q.shape[0]})")
        actual_max_q = int(q_lens.max().item())
        if max_seqlen_q < actual_max_q:
            raise ValueError(f"max_seqlen_q ({max_seqlen_q}) must be >= actual max Q "
                             f"sequence length ({actual_max_q})")
        if int(cache_seqlens.min().item()) < 0:
            raise ValueError("cache_seqlens must be non-negative")
        max_total_len = int((cache_seqlens + q_lens).max().item())
        if max_total_len > self.max_cache_len:
            raise ValueError("cache_seqlens + q_len exceeds paged KV capacity: "
                             f"max total length {max_total_len}, capacity {self.max_cache_len}")
        if self.fuse_rope and max_total_len > self.max_position:
            raise ValueError("cache_seqlens + q_len exceeds RoPE max_position: "
                             f"max total length {max_total_len}, max_position {self.max_position}")
        num_pages = k_pages.shape[0] // self.page_size
        if int(block_table.min().item()) < 0:
            raise ValueError("block_table must contain non-negative physical page ids")
        max_page = int(block_table.max().item())
        if max_page >= num_pages:
            raise ValueError(f"block_table references page {max_page}, but only {num_pages} pages exist")

    def _infer_output_shapes(self, q_shape, *rest) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q, cache_seqlens,
                block_table, max_seqlen_q) -> torch.Tensor:
        self._validate_forward_inputs(q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q,
                                      cache_seqlens, block_table, max_seqlen_q)
        self.dtype = q.dtype
        call = self.attention_call(q.dtype)
        key = self.select_kernel_key(PAGED_PREFILL_KEYS, call)
        inputs = (q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q, cache_seqlens, block_table)
        cos_table, sin_table = self._get_rope_cos_sin(q.device, q.dtype) if self.fuse_rope else (None, None)
        return self._get_kernel(inputs, key, call)(*inputs, max_seqlen_q, cos_table, sin_table)

    def _get_rope_cos_sin(self, device: torch.device, dtype: torch.dtype):
        """cos / sin tables ``[max_position, rotary_dim / 2]`` in the attention element type, computed in
        fp32 as the reference's ``base_freqs`` does (``src/tileops/ops/rope.py:97-120``); cached."""
        cached = self._rope_tables.get((device, dtype))
        if cached is None:
            half = self.rotary_dim // 2
            freqs = 1.0 / (self.rope_base ** (torch.arange(0, half, device=device, dtype=torch.float32) / half))
            angles = torch.outer(torch.arange(self.max_position, device=device, dtype=torch.float32), freqs)
            cached = (torch.cos(angles).to(dtype), torch.sin(angles).to(dtype))
            self._rope_tables[(device, dtype)] = cached
        return cached

    @property
    def total_flops(self) -> int:
        raise NotImplementedError("total_flops is not defined for paged varlen ops; "
                                  "compute per-sample from cu_seqlens and cache_seqlens at call time.")

    @property
    def total_memory(self) -> int:
        raise NotImplementedError("total_memory is not defined for paged varlen ops; "
                                  "compute per-sample from cu_seqlens and cache_seqlens at call time.")


def _validate_windows(window_size_left: int, window_size_right: int) -> None:
    if window_size_left != -1 and window_size_left < 0:
        raise ValueError(f"window_size_left must be -1 (unlimited) or >= 0, got {window_size_left}")
    if window_size_right != -1 and window_size_right < 0:
        raise ValueError(f"window_size_right must be -1 (unlimited) or >= 0, got {window_size_right}")


class GroupedQueryAttentionSlidingWindowFwdOp(Op):
    """Fixed-length GQA forward with sliding-window attention (BSHD, Sq == Skv).  Row ``q_pos`` sees
    key ``k_pos`` iff ``k_pos <= q_pos`` (causal), ``k_pos >= q_pos - window_size_left`` (when >= 0) and
    ``k_pos <= q_pos + window_size_right`` (when >= 0).  Mirrors
    ``src/tileops/ops/attention/gqa.py:1457-1627`` of the reference."""

    def __init__(self, batch: int, heads: int, heads_kv: int, seq_len: int, dim: int, is_causal: bool = True,
                 window_size_left: int = -1, window_size_right: int = -1,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        if heads % heads_kv != 0:
            raise ValueError("heads must be divisible by heads_kv")
        _validate_windows(window_size_left, window_size_right)
        self.batch, self.heads, self.heads_kv, self.seq_len, self.dim = batch, heads, heads_kv, seq_len, dim
        self.is_causal = is_causal
        self.window_size_left, self.window_size_right = window_size_left, window_size_right
        self.dtype = None
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_sliding_window_fwd_kernel": GQASlidingWindowSm100Kernel}

    def _get_kernel(self, inputs, dtype: torch.dtype) -> Kernel:
        return self.get_or_build_kernel(
            "gqa_sliding_window_fwd_kernel", inputs, key=dtype,
            build=lambda: self.kernel_map["gqa_sliding_window_fwd_kernel"](
                batch=self.batch, heads=self.heads, heads_kv=self.heads_kv, seq_len=self.seq_len, dim=self.dim,
                is_causal=self.is_causal, window_size_left=self.window_size_left,
                window_size_right=self.window_size_right, dtype=dtype, tune=self.tune))

    def _infer_output_shapes(self, q_shape, k_shape, v_shape) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        for t, name in ((q, "q"), (k, "k"), (v, "v")):
            if t.device.type != "cuda":
                raise ValueError(f"{name} must be on a cuda device, got {t.device}")
            if t.dtype != q.dtype:
                raise ValueError(f"{name} dtype {t.dtype} does not match q dtype {q.dtype}")
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        want_q = (self.batch, self.seq_len, self.heads, self.dim)
        want_kv = (self.batch, self.seq_len, self.heads_kv, self.dim)
        if tuple(q.shape) != want_q:
            raise ValueError(f"q shape {q.shape} does not match expected {want_q}")
        if tuple(k.shape) != want_kv:
            raise ValueError(f"k shape {k.shape} does not match expected {want_kv}")
        if tuple(v.shape) != want_kv:
            raise ValueError(f"v shape {v.shape} does not match expected {want_kv}")
        self.dtype = q.dtype
        return self._get_kernel((q, k, v), q.dtype).forward(q, k, v)

    @property
    def total_flops(self) -> int:
        S, wl, wr = self.seq_len, self.window_size_left, self.window_size_right
        attended = 0
        for i in range(S):
            hi = i if self.is_causal else (min(S - 1, i + wr) if wr >= 0 else S - 1)
            lo = max(0, i - wl) if wl >= 0 else 0
            attended += hi - lo + 1
        return 4 * self.batch * self.heads * attended * self.dim

    @property
    def total_memory(self) -> int:
        if self.dtype is None:
            raise RuntimeError(f"{type(self).__name__}.total_memory requires a prior forward() "
                               "call to bind the element type")
        return 2 * self.batch * self.seq_len * (self.heads + self.heads_kv) * self.dim * self.dtype.itemsize

    def eval_roofline(self) -> tuple:
        return self.total_flops, self.total_memory


class GroupedQueryAttentionSlidingWindowVarlenFwdOp(Op):
    """Packed GQA forward with sliding-window attention; per request, with
    ``offset = seqlen_k - seqlen_q`` (bottom-right), row ``q_pos`` sees ``k_pos`` iff
    ``k_pos <= q_pos + offset`` (causal), ``k_pos >= q_pos + offset - window_size_left`` (when >= 0) and
    ``k_pos <= q_pos + offset + window_size_right`` (when >= 0).  Mirrors
    ``src/tileops/ops/attention/gqa.py:1630-1831`` of the reference."""

    def __init__(self, batch: int, heads: int, heads_kv: int, dim: int, is_causal: bool = True,
                 window_size_left: int = -1, window_size_right: int = -1,
                 accum_dtype: torch.dtype = torch.float32,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        if heads % heads_kv != 0:
            raise ValueError("heads must be divisible by heads_kv")
        _validate_windows(window_size_left, window_size_right)
        self.batch, self.heads, self.heads_kv, self.dim = batch, heads, heads_kv, dim
        self.is_causal = is_causal
        self.window_size_left, self.window_size_right = window_size_left, window_size_right
        self.accum_dtype = accum_dtype
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"gqa_sliding_window_varlen_fwd_kernel": GQASlidingWindowVarlenSm100Kernel}

    def _get_kernel(self, inputs, dtype: torch.dtype, max_seqlen_q: int) -> Kernel:
        return self.get_or_build_kernel(
            "gqa_sliding_window_varlen_fwd_kernel", inputs, key=(dtype, max_seqlen_q),
            build=lambda: self.kernel_map["gqa_sliding_window_varlen_fwd_kernel"](
                batch=self.batch, heads=self.heads, heads_kv=self.heads_kv, max_seqlen_q=max_seqlen_q,
                max_seqlen_kv=max_seqlen_q, dim=self.dim, is_causal=self.is_causal, dtype=dtype,
                window_size_left=self.window_size_left, window_size_right=self.window_size_right,
                accum_dtype=self.accum_dtype, tune=self.tune))

    def _infer_output_shapes(self, q_shape, *rest) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q: int) -> torch.Tensor:
        for t, name in ((q, "q"), (k, "k"), (v, "v")):
            if t.device.type != "cuda":
                raise ValueError(f"{name} must be on a cuda device, got {t.device}")
            if t.dtype != q.dtype:
                raise ValueError(f"{name} dtype {t.dtype} does not match q dtype {q.dtype}")
            if not t.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        if q.ndim != 3 or q.shape[1] != self.heads or q.shape[2] != self.dim:
            raise ValueError(f"q shape {q.shape} incompatible with heads={self.heads}, dim={self.dim}")
        for t, name in ((k, "k"), (v, "v")):
            if t.ndim != 3 or t.shape[1] != self.heads_kv or t.shape[2] != self.dim:
                raise ValueError(f"{name} shape {t.shape} incompatible with heads_kv={self.heads_kv}, dim={self.dim}")
        for cu, name in ((cu_seqlens_q, "cu_seqlens_q"), (cu_seqlens_k, "cu_seqlens_k")):
            if cu.shape[0] != self.batch + 1:
                raise ValueError(f"{name}.shape[0] ({cu.shape[0]}) must equal batch+1 ({self.batch + 1})")
        for cu, name in ((cu_seqlens_q, "cu_seqlens_q"), (cu_seqlens_k, "cu_seqlens_k")):
            if cu.device.type != "cuda":
                raise ValueError(f"{name} must be on a cuda device, got {cu.device}")
            if cu.dtype != torch.int32:
                raise ValueError(f"{name} must have dtype int32, got {cu.dtype}")
            if not cu.is_contiguous():
                raise ValueError(f"{name} must be contiguous")
        for cu, name in ((cu_seqlens_q, "cu_seqlens_q"), (cu_seqlens_k, "cu_seqlens_k")):
            if cu[0].item() != 0:
                raise ValueError(f"{name}[0] must be 0, got {cu[0].item()}")
        for cu, name in ((cu_seqlens_q, "cu_seqlens_q"), (cu_seqlens_k, "cu_seqlens_k")):
            if not torch.all(cu[1:] >= cu[:-1]):
                raise ValueError(f"{name} must be non-decreasing")
        if cu_seqlens_q[-1].item() > q.shape[0]:
            raise ValueError(f"cu_seqlens_q[-1] ({cu_seqlens_q[-1].item()}) exceeds q.shape[0] ({q.shape[0]})")
        if cu_seqlens_k[-1].item() > k.shape[0]:
            raise ValueError(f"cu_seqlens_k[-1] ({cu_seqlens_k[-1].item()}) exceeds k.shape[0] ({k.shape[0]})")
        actual_max_q = int((cu_seqlens_q[1:] - cu_seqlens_q[:-1]).max().item())
        if max_seqlen_q < actual_max_q:
            raise ValueError(f"max_seqlen_q ({max_seqlen_q}) must be >= actual max Q "
                             f"sequence length ({actual_max_q})")
        self.dtype = q.dtype
        return self._get_kernel((q, k, v, cu_seqlens_q, cu_seqlens_k), q.dtype, max_seqlen_q).forward(
            q, k, v, cu_seqlens_q, cu_seqlens_k)

    @property
    def total_flops(self) -> int:
        raise NotImplementedError("total_flops is not defined for varlen ops; "
                                  "compute per-sample from cu_seqlens at call time.")

    @property
    def total_memory(self) -> int:
        raise NotImplementedError("total_memory is not defined for varlen ops; "
                                  "compute per-sample from cu_seqlens at call time.")


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
    ``[seqlen_kv, heads_kv, dim]``; real_seqlen_kv ``[B]`` int32; block_table ``[B, num_pages]`` int32.

    The kernel trusts the block table (a wrong page id is an out-of-bounds read).  Setting the attribute
    ``validate_inputs = True`` on an instance makes every ``forward`` check lengths and page ids on the host
    first, the check the reference's paged prefill does on every call
    (``src/tileops/ops/attention/gqa.py:1038-1046``); it reads both tensors back, so it is off by default
    and stays off on a timed path."""

    _KEYS = PAGED_DECODE_KEYS
    validate_inputs = False

    def _check_table(self, k: torch.Tensor, real_seqlen_kv: torch.Tensor, block_table: torch.Tensor) -> None:
        """Host-side range check of lengths and the page ids they reach (synchronises)."""
        lens = real_seqlen_kv.detach().cpu().to(torch.int64)
        table = block_table.detach().cpu().to(torch.int64)
        width = table.shape[1]
        pool_pages = k.shape[0] // self.page_size
        if bool((lens < 0).any()):
            raise ValueError("real_seqlen_kv must be non-negative")
        need = (lens + self.page_size - 1) // self.page_size
        if bool((need > width).any()):
            b = int((need > width).nonzero()[0])
            raise ValueError(f"real_seqlen_kv[{b}]={int(lens[b])} needs {int(need[b])} pages, block_table has {width}")
        live = torch.arange(width)[None, :] < need[:, None]
        bad = live & ((table < 0) | (table >= pool_pages))
        if bool(bad.any()):
            b, i = (int(x) for x in bad.nonzero()[0])
            raise ValueError(f"block_table[{b}, {i}]={int(table[b, i])} is outside the pool of {pool_pages} pages")

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
        if self.validate_inputs:
            self._check_table(k, real_seqlen_kv, block_table)
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
        if self.validate_inputs:
            self._check_table(k, real_seqlen_kv, block_table)
        return self._get_kernel((q, k, v, k_scale, v_scale, real_seqlen_kv, block_table), q.dtype)(
            q, k, v, k_scale, v_scale, real_seqlen_kv, block_table)

    def eval_roofline(self) -> tuple:
        from ..perf.formulas import gqa_decode_paged_roofline
        data = dict(vars(self))
        data["dtype"] = getattr(self, "cache_dtype", None) or fp8_dtype()
        return gqa_decode_paged_roofline(data)
