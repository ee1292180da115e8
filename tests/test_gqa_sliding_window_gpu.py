"""GPU parity of sliding-window prefill (fixed length and packed) against the fp32 oracle and the
golden vectors produced by the reference tests' reference programs.  Cases follow
``tests/ops/attention/test_gqa_sliding_window.py`` / ``test_gqa_sliding_window_varlen.py`` of the
reference (windows, head ratios, sequence lengths)."""

import os

import numpy as np
import pytest
import torch

from oracle import gqa_oracle as O

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
TOL = {torch.float16: dict(atol=5e-3, rtol=1e-2), torch.bfloat16: dict(atol=2e-2, rtol=1e-2)}


@pytest.mark.parametrize("batch,seq,heads,heads_kv,dim,causal,wl,wr,dtype", [
    (2, 512, 8, 2, 64, True, -1, -1, torch.float16),
    (2, 512, 8, 2, 64, True, 128, -1, torch.float16),
    (2, 512, 8, 2, 64, False, 64, 64, torch.float16),
    (2, 128, 8, 1, 128, True, 1, -1, torch.float16),
    (2, 512, 8, 2, 64, False, 64, 64, torch.bfloat16),
    (2, 768, 8, 2, 64, False, 256, -1, torch.float16),
    (1, 2048, 8, 2, 64, True, 512, -1, torch.float16),
    (2, 512, 8, 2, 64, False, -1, 64, torch.float16),
    (2, 256, 8, 2, 64, True, 0, -1, torch.float16),
    (1, 1000, 4, 4, 128, True, 77, -1, torch.bfloat16),
    (1, 1000, 4, 2, 128, False, 200, 3, torch.bfloat16),
])
def test_sliding_window_fwd_op(batch, seq, heads, heads_kv, dim, causal, wl, wr, dtype):
    from tileops_b200.ops import GroupedQueryAttentionSlidingWindowFwdOp
    g = torch.Generator().manual_seed(1235)
    q = torch.randn(batch, seq, heads, dim, generator=g).to(dtype)
    k = torch.randn(batch, seq, heads_kv, dim, generator=g).to(dtype)
    v = torch.randn(batch, seq, heads_kv, dim, generator=g).to(dtype)
    op = GroupedQueryAttentionSlidingWindowFwdOp(batch=batch, heads=heads, heads_kv=heads_kv, seq_len=seq, dim=dim,
                                                 is_causal=causal, window_size_left=wl, window_size_right=wr)
    o = op(q.cuda(), k.cuda(), v.cuda())
    ref = O.prefill_ref(q, k, v, causal, window_left=wl, window_right=wr)
    torch.testing.assert_close(o.cpu().float(), ref.float(), **TOL[dtype])
    assert op.total_flops > 0 and op.total_memory > 0


@pytest.mark.parametrize("sq,sk,causal,wl,wr", [
    ([128, 64], [128, 64], True, 32, -1),
    ([100, 37, 300], [100, 37, 300], True, 64, -1),
    ([64, 200], [300, 200], True, 50, -1),        # kv longer than q: bottom-right offset
    ([130, 90], [260, 400], False, 40, 25),
    ([1, 257], [500, 257], True, -1, -1),
    ([150, 150], [150, 150], False, -1, 10),
])
def test_sliding_window_varlen_op(sq, sk, causal, wl, wr):
    from tileops_b200.ops import GroupedQueryAttentionSlidingWindowVarlenFwdOp
    g = torch.Generator().manual_seed(77)
    H, Hkv, D = 8, 2, 128
    cu_q = torch.tensor([0] + list(np.cumsum(sq)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(np.cumsum(sk)), dtype=torch.int32)
    q = torch.randn(sum(sq), H, D, generator=g).half()
    k = torch.randn(sum(sk), Hkv, D, generator=g).half()
    v = torch.randn(sum(sk), Hkv, D, generator=g).half()
    op = GroupedQueryAttentionSlidingWindowVarlenFwdOp(batch=len(sq), heads=H, heads_kv=Hkv, dim=D, is_causal=causal,
                                                       window_size_left=wl, window_size_right=wr)
    o = op(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), max(sq))
    ref = O.prefill_packed_ref(q, k, v, cu_q, cu_k, causal, window_left=wl, window_right=wr)
    torch.testing.assert_close(o.cpu().float(), ref.float(), **TOL[torch.float16])


def test_packed_op_routes_windows_to_the_sliding_window_kernel():
    from tileops_b200.ops import GroupedQueryAttentionPrefillFwdOp
    g = torch.Generator().manual_seed(78)
    B, S, H, Hkv, D = 2, 256, 8, 2, 128
    q = torch.randn(B * S, H, D, generator=g).bfloat16()
    k = torch.randn(B * S, Hkv, D, generator=g).bfloat16()
    v = torch.randn(B * S, Hkv, D, generator=g).bfloat16()
    cu = (torch.arange(B + 1, dtype=torch.int32) * S)
    op = GroupedQueryAttentionPrefillFwdOp(B, H, Hkv, D, S, S, dtype=torch.bfloat16, is_causal=True,
                                           window_size_left=100)
    ones = torch.ones(B, Hkv, device="cuda")
    o = op(q.cuda(), k.cuda(), v.cuda(), cu.cuda(), cu.cuda(), ones, ones.clone(), ones.clone())
    ref = O.prefill_packed_ref(q, k, v, cu, cu, True, window_left=100)
    torch.testing.assert_close(o.cpu().float(), ref.float(), **TOL[torch.bfloat16])


def test_golden_vectors():
    from tileops_b200 import functional as F
    G = np.load(os.path.join(HERE, "golden", "gqa_golden.npz"))

    def pad(x):   # the fixtures are D = 32; zero columns change neither scores nor outputs
        x = torch.from_numpy(x)
        return torch.cat([x, torch.zeros_like(x)], dim=-1).half().cuda()
    q, k, v = pad(G["sw_q"]), pad(G["sw_k"]), pad(G["sw_v"])
    for name, (causal, wl, wr) in {"c_l17": (True, 17, -1), "n_l8_r5": (False, 8, 5), "n_r11": (False, -1, 11),
                                   "c_l0": (True, 0, -1)}.items():
        o = F.gqa_prefill(q, k, v, is_causal=causal, sm_scale=32 ** -0.5, window_size_left=wl, window_size_right=wr)
        torch.testing.assert_close(o[..., :32].cpu().float(), torch.from_numpy(G["sw_o_" + name]), atol=5e-3, rtol=1e-2)
    q, k, v = pad(G["swv_q"]), pad(G["swv_k"]), pad(G["swv_v"])
    cu_q, cu_k = torch.from_numpy(G["swv_cu_q"]).cuda(), torch.from_numpy(G["swv_cu_k"]).cuda()
    for name, (causal, wl, wr) in {"c_l9": (True, 9, -1), "n_l4_r6": (False, 4, 6)}.items():
        o = F.gqa_prefill_paged(q, k, v, None, None, cu_q, None, None, 24, is_causal=causal, sm_scale=32 ** -0.5,
                                cu_seqlens_kv=cu_k, window_size_left=wl, window_size_right=wr)
        torch.testing.assert_close(o[..., :32].cpu().float(), torch.from_numpy(G["swv_o_" + name]), atol=5e-3, rtol=1e-2)
