"""MHA decode operators: same names, constructors and ``forward`` signatures as the reference's
``MultiHeadAttentionDecodeWithKVCacheFwdOp`` and ``MultiHeadAttentionDecodePagedWithKVCacheFwdOp``
(``src/tileops/ops/attention/mha.py:194-346``), served by the GQA decode kernel with one q head per KV
head.  The contiguous op does not pad K/V up to ``seqlen_kv`` (the reference copies them with ``F.pad``):
the live length is a kernel argument."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..kernels.call_spec import AttentionCall
from ..kernels.kernel_base import Kernel
from ..kernels.mha_decode import MHADecodePagedSm100Kernel, MHADecodeSm100Kernel
from .op_base import Op

__all__ = ["MultiHeadAttentionDecodeWithKVCacheFwdOp", "MultiHeadAttentionDecodePagedWithKVCacheFwdOp",
           "MHA_PAGED_DECODE_KEYS"]

MHA_PAGED_DECODE_KEYS = ("mha_decode_paged_ws_kernel", "mha_decode_paged_kernel")


class MultiHeadAttentionDecodeWithKVCacheFwdOp(Op):
    """Layout: BSHD.  q ``[B, Sq, H, D]``, k/v ``[B, S, H, D]`` with ``S <= seqlen_kv`` live tokens."""

    def __init__(self, batch: int, heads: int, seqlen_q: int, seqlen_kv: int, dim: int,
                 kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        self.batch, self.heads, self.seqlen_q, self.seqlen_kv, self.dim = batch, heads, seqlen_q, seqlen_kv, dim
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"mha_decode_kernel": MHADecodeSm100Kernel}

    def _get_kernel(self, inputs, dtype: torch.dtype) -> Kernel:
        return self.get_or_build_kernel(
            "mha_decode_kernel", inputs, key=dtype,
            build=lambda: self.kernel_map["mha_decode_kernel"](
                self.batch, self.heads, self.seqlen_q, self.seqlen_kv, self.dim, False, dtype, tune=self.tune))

    def _infer_output_shapes(self, q_shape, k_shape, v_shape) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        real_seqlen_kv = k.shape[1]
        if real_seqlen_kv > self.seqlen_kv:
            raise ValueError(f"k holds {real_seqlen_kv} tokens, more than seqlen_kv={self.seqlen_kv}")
        self.dtype = q.dtype
        return self._get_kernel((q, k, v), q.dtype)(q, k, v, real_seqlen_kv)


class MultiHeadAttentionDecodePagedWithKVCacheFwdOp(Op):
    """Paged MHA decode.  q ``[B, Sq, H, D]``; k, v physical pool ``[seqlen_kv, H, D]``; real_seqlen_kv
    ``[B]`` int32; block_table ``[B, num_pages]`` int32."""

    def __init__(self, batch: int, heads: int, seqlen_q: int, seqlen_kv: int, dim: int, page_size: int,
                 is_causal: bool = False, kernel_map: Optional[Dict[str, type]] = None, tune: bool = False) -> None:
        self.batch, self.heads, self.seqlen_q, self.seqlen_kv, self.dim = batch, heads, seqlen_q, seqlen_kv, dim
        self.page_size, self.is_causal = page_size, is_causal
        self.tune = tune
        self.dispatch_kernel(kernel_map)

    @property
    def default_kernel_map(self) -> Dict[str, type]:
        return {"mha_decode_paged_kernel": MHADecodePagedSm100Kernel}

    def _attention_call(self, dtype: torch.dtype) -> AttentionCall:
        return AttentionCall(dtype=dtype, batch=self.batch, heads=self.heads, heads_kv=self.heads, dim=self.dim,
                             max_seqlen_q=self.seqlen_q, seqlen_kv=self.seqlen_kv, page_size=self.page_size,
                             is_causal=self.is_causal, tune=self.tune)

    def _get_kernel(self, inputs, dtype: torch.dtype) -> Kernel:
        call = self._attention_call(dtype)
        key = self.select_kernel_key(MHA_PAGED_DECODE_KEYS, call)
        return self.get_or_build_kernel(key, inputs, key=dtype, build=lambda: self.kernel_map[key](
            call.batch, call.heads, call.max_seqlen_q, call.seqlen_kv, call.dim, call.page_size, call.is_causal,
            dtype, tune=call.tune))

    def _infer_output_shapes(self, q_shape, k_shape, v_shape, real_seqlen_kv_shape,
                             block_table_shape) -> Dict[str, tuple]:
        return {"o": tuple(q_shape)}

    def forward(self, q, k, v, real_seqlen_kv, block_table) -> torch.Tensor:
        self.dtype = q.dtype
        return self._get_kernel((q, k, v, real_seqlen_kv, block_table), q.dtype)(
            q, k, v, real_seqlen_kv, block_table)
