"""sm_100a kernel classes for MHA decode: the ``heads_kv == heads`` case of the GQA decode kernel.

Slots and constructors of the reference's ``MHADecodeKernel`` / ``MHADecodePagedKernel`` as
``MultiHeadAttentionDecode{,Paged}WithKVCacheFwdOp`` build them
(``src/tileops/ops/attention/mha.py:212-226,284-301``): q is ``[batch, seqlen_q, heads, dim]``.  With
``seqlen_q == 1`` the call is GQA decode with one q head per KV head.  With ``seqlen_q > 1`` and no causal
mask the ``seqlen_q`` rows of a head share that head's K/V exactly like the q heads of a GQA group, so
they are laid out as a group of ``seqlen_q`` heads (a small host-side permute of q and o) and the same
CUDA kernel runs.  The paged kernel's causal mask between the rows of a call is the reference's top-left
aligned one (``src/tileops/kernels/attention/mha_decode_paged.py:72-95``: row ``i`` sees keys ``0..i``): every
(sequence, row) then becomes a sequence of its own with length ``min(i + 1, real_seqlen_kv)`` over the same
pages, again one launch of the same kernel.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import functional as F
from .call_spec import ATTENTION_DTYPES
from .kernel_base import Kernel

__all__ = ["MHADecodeSm100Kernel", "MHADecodePagedSm100Kernel"]


def _as_groups(q: torch.Tensor) -> torch.Tensor:
    """[B, Sq, H, D] -> [B, H * Sq, D]: head h's rows become the q-head group of KV head h."""
    B, Sq, H, D = q.shape
    if Sq == 1:
        return q.reshape(B, H, D)
    return q.permute(0, 2, 1, 3).reshape(B, H * Sq, D)


def _from_groups(o: torch.Tensor, B: int, Sq: int, H: int, D: int) -> torch.Tensor:
    if Sq == 1:
        return o.view(B, 1, H, D)
    return o.view(B, H, Sq, D).permute(0, 2, 1, 3).contiguous()


class _MHADecodeBase(Kernel):
    supported_archs = [100]
    general = True
    #: whether a causal mask between several q rows of one call is served (the paged kernel only)
    serves_causal_rows = False

    @classmethod
    def applies(cls, call) -> bool:
        return (call.dim in (64, 128) and call.dtype in ATTENTION_DTYPES
                and (cls.serves_causal_rows or not (call.is_causal and call.max_seqlen_q > 1)))

    def _common(self, batch, heads, seqlen_q, seqlen_kv, dim, is_causal, dtype, tune):
        if dim not in (64, 128):
            raise ValueError(f"{type(self).__name__} supports head dim 64 and 128, got {dim}")
        if is_causal and seqlen_q > 1 and not self.serves_causal_rows:
            raise ValueError(f"{type(self).__name__} does not serve a causal mask between the q rows")
        self.batch, self.heads, self.seqlen_q, self.seqlen_kv, self.dim = batch, heads, seqlen_q, seqlen_kv, dim
        self.is_causal, self.dtype, self.tune = is_causal, dtype, tune


class MHADecodeSm100Kernel(_MHADecodeBase):
    """Contiguous cache: ``forward(Q[B,Sq,H,D], K[B,S,H,D], V, real_seqlen_kv: int)``."""

    def __init__(self, batch, heads, seqlen_q, seqlen_kv, dim, is_causal, dtype, config: Optional[dict] = None,
                 tune: bool = False, device_index=None) -> None:
        super().__init__(device_index=device_index)
        self._common(batch, heads, seqlen_q, seqlen_kv, dim, is_causal, dtype, tune)
        self.init_config(config, tune)

    def forward(self, Q, K, V, real_seqlen_kv=None):
        self._require_cuda(Q=Q, K=K, V=V)
        B, Sq, H, D = Q.shape
        live = K.shape[1] if real_seqlen_kv is None else real_seqlen_kv
        o = F.gqa_decode(_as_groups(Q), K, V, real_seqlen_kv=live)
        return _from_groups(o, B, Sq, H, D)


class MHADecodePagedSm100Kernel(_MHADecodeBase):
    """Paged cache: ``forward(Q[B,Sq,H,D], K[N,H,D], V, real_seqlen_kv[B] i32, block_table[B,W] i32)``."""

    serves_causal_rows = True

    def __init__(self, batch, heads, seqlen_q, seqlen_kv, dim, page_size, is_causal, dtype,
                 config: Optional[dict] = None, tune: bool = False, device_index=None) -> None:
        super().__init__(device_index=device_index)
        self._common(batch, heads, seqlen_q, seqlen_kv, dim, is_causal, dtype, tune)
        if seqlen_kv % page_size != 0:
            raise ValueError(f"seqlen_kv={seqlen_kv} must be a multiple of page_size={page_size}")
        self.page_size = page_size
        self.init_config(config, tune)

    def forward(self, Q, K, V, real_seqlen_kv, block_table):
        self._require_cuda(Q=Q, K=K, V=V, real_seqlen_kv=real_seqlen_kv, block_table=block_table)
        B, Sq, H, D = Q.shape
        if self.is_causal and Sq > 1:
            # row i of sequence b: a sequence of its own that sees keys 0..i of b's pages (no host sync)
            rows = torch.arange(1, Sq + 1, device=Q.device, dtype=torch.int32).repeat(B)
            lens = torch.minimum(real_seqlen_kv.repeat_interleave(Sq), rows)
            o = F.gqa_decode(Q.reshape(B * Sq, H, D), K, V, real_seqlen_kv=lens,
                             block_table=block_table.repeat_interleave(Sq, dim=0), page_size=self.page_size)
            return o.view(B, Sq, H, D)
        o = F.gqa_decode(_as_groups(Q), K, V, real_seqlen_kv=real_seqlen_kv, block_table=block_table,
                         page_size=self.page_size)
        return _from_groups(o, B, Sq, H, D)
