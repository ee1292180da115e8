"""GPU parity of the MHA decode ops (the heads_kv == heads case of the decode kernel) against the oracle.
Cases follow ``tests/ops/attention/test_mha_decode.py`` / ``test_mha_decode_paged.py`` of the reference
(seqlen_q = 1, no causal mask), plus multi-row q, which the reference op signature also admits."""

import pytest
import torch

from oracle import gqa_oracle as O

pytestmark = pytest.mark.gpu
ATOL = {torch.float16: 2e-3, torch.bfloat16: 1e-2}


def _ref(q, k, v):
    """q [B,Sq,H,D], k/v [B,S,H,D] (logical) -> [B,Sq,H,D]: non-causal attention per head, which is
    what the reference's scaled_dot_product_attention reference programs compute."""
    B, Sq, H, D = q.shape
    o = O.decode_ref(q.permute(0, 2, 1, 3).reshape(B, H * Sq, D), k, v)
    return o.view(B, H, Sq, D).permute(0, 2, 1, 3)


@pytest.mark.parametrize("batch,heads,seqlen_q,seqlen_kv,dim,page,dtype", [
    (1, 16, 1, 512, 128, 128, torch.float16),
    (1, 16, 1, 1024, 128, 128, torch.bfloat16),
    (1, 8, 1, 1024, 64, 256, torch.float16),
    (2, 8, 1, 1024, 64, 256, torch.float16),
    (3, 8, 4, 1024, 128, 64, torch.bfloat16),
])
def test_mha_decode_paged_op(batch, heads, seqlen_q, seqlen_kv, dim, page, dtype):
    from tileops_b200.ops import MultiHeadAttentionDecodePagedWithKVCacheFwdOp
    g = torch.Generator().manual_seed(5)
    pages = seqlen_kv // page
    lens = torch.randint(page, pages * page // batch + 1, (batch,), generator=g).to(torch.int32)
    per = pages // batch
    bt = torch.randperm(pages, generator=g).to(torch.int32)[: batch * per].reshape(batch, per)
    q = torch.randn(batch, seqlen_q, heads, dim, generator=g).to(dtype)
    k = torch.randn(seqlen_kv, heads, dim, generator=g).to(dtype)
    v = torch.randn(seqlen_kv, heads, dim, generator=g).to(dtype)
    op = MultiHeadAttentionDecodePagedWithKVCacheFwdOp(batch, heads, seqlen_q, seqlen_kv, dim, page)
    o = op(q.cuda(), k.cuda(), v.cuda(), lens.cuda(), bt.cuda())
    assert o.shape == q.shape and o.dtype == dtype
    for b in range(batch):
        rows = torch.from_numpy(O.physical_rows(bt[b].numpy(), int(lens[b]), page))
        ref = _ref(q[b:b + 1], k[rows].unsqueeze(0), v[rows].unsqueeze(0))
        torch.testing.assert_close(o[b:b + 1].cpu().float(), ref.float(), atol=ATOL[dtype], rtol=1e-2)


@pytest.mark.parametrize("batch,heads,seqlen_q,seqlen_kv,live,dim,dtype", [
    (1, 32, 1, 8192, 8192, 128, torch.float16),
    (4, 16, 1, 2048, 1500, 128, torch.bfloat16),
    (2, 8, 3, 512, 300, 64, torch.float16),
])
def test_mha_decode_op(batch, heads, seqlen_q, seqlen_kv, live, dim, dtype):
    from tileops_b200.ops import MultiHeadAttentionDecodeWithKVCacheFwdOp
    g = torch.Generator().manual_seed(6)
    q = torch.randn(batch, seqlen_q, heads, dim, generator=g).to(dtype)
    k = torch.randn(batch, live, heads, dim, generator=g).to(dtype)
    v = torch.randn(batch, live, heads, dim, generator=g).to(dtype)
    op = MultiHeadAttentionDecodeWithKVCacheFwdOp(batch, heads, seqlen_q, seqlen_kv, dim)
    o = op(q.cuda(), k.cuda(), v.cuda())
    torch.testing.assert_close(o.cpu().float(), _ref(q, k, v).float(), atol=ATOL[dtype], rtol=1e-2)


def test_causal_multi_row_q_is_refused():
    from tileops_b200.ops import MultiHeadAttentionDecodePagedWithKVCacheFwdOp
    op = MultiHeadAttentionDecodePagedWithKVCacheFwdOp(1, 8, 4, 512, 128, 64, is_causal=True)
    q = torch.zeros(1, 4, 8, 128, device="cuda", dtype=torch.float16)
    k = torch.zeros(512, 8, 128, device="cuda", dtype=torch.float16)
    with pytest.raises(ValueError, match="no implementation serves this call"):
        op(q, k, k, torch.full((1,), 64, dtype=torch.int32, device="cuda"),
           torch.zeros(1, 8, dtype=torch.int32, device="cuda"))
