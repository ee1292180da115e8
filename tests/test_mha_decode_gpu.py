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


def test_causal_multi_row_paged_decode_matches_the_reference_mask():
    """The reference's paged MHA decode masks top-left aligned (row i sees keys 0..i,
    src/tileops/kernels/attention/mha_decode_paged.py:72-95); rows are clamped to the live length."""
    from tileops_b200.ops import MultiHeadAttentionDecodePagedWithKVCacheFwdOp
    B, H, Sq, D, page, pool = 2, 8, 4, 128, 64, 512
    g = torch.Generator().manual_seed(8)
    q = torch.randn(B, Sq, H, D, generator=g).to(torch.float16)
    k = torch.randn(pool, H, D, generator=g).to(torch.float16)
    v = torch.randn(pool, H, D, generator=g).to(torch.float16)
    lens = torch.tensor([200, 3], dtype=torch.int32)                  # the second sequence is shorter than Sq
    bt = torch.randperm(pool // page, generator=g).to(torch.int32).reshape(B, -1)
    op = MultiHeadAttentionDecodePagedWithKVCacheFwdOp(B, H, Sq, pool, D, page, is_causal=True)
    o = op(q.cuda(), k.cuda(), v.cuda(), lens.cuda(), bt.cuda()).cpu().float()
    for b in range(B):
        rows = torch.from_numpy(O.physical_rows(bt[b].numpy(), int(lens[b]), page))
        kb, vb = k[rows].float(), v[rows].float()
        for i in range(Sq):
            n = min(i + 1, int(lens[b]))
            sc = torch.einsum("hd,nhd->hn", q[b, i].float(), kb[:n]) * D ** -0.5
            ref = torch.einsum("hn,nhd->hd", torch.softmax(sc, -1), vb[:n])
            torch.testing.assert_close(o[b, i], ref, atol=5e-3, rtol=1e-2)


def test_causal_multi_row_contiguous_decode_is_refused():
    from tileops_b200.kernels.mha_decode import MHADecodeSm100Kernel
    with pytest.raises(ValueError, match="causal mask between the q rows"):
        MHADecodeSm100Kernel(1, 8, 4, 512, 128, True, torch.float16)
