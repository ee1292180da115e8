"""GPU parity of the packed paged-cache prefill (tcgen05 kernel, C ABI ``tb200_gqa_prefill_paged``)
against the fp32 oracle and the committed golden vectors.  The cases mirror the reference's
``tests/ops/attention/test_gqa_prefill_paged.py`` (lengths, head ratios, page sizes)."""

import os

import numpy as np
import pytest
import torch

from oracle import gqa_oracle as O

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
TOL = {torch.float16: dict(atol=5e-3, rtol=1e-3), torch.bfloat16: dict(atol=2e-2, rtol=1e-2)}


def _F():
    from tileops_b200 import functional as F
    return F


def _case(q_lens, old_lens, heads, heads_kv, dim, page, dtype, seed=0, pool_fill=0.0, pages_per_req=None):
    g = torch.Generator().manual_seed(1235 + seed)
    nb = len(q_lens)
    W = pages_per_req or max((o + q + page - 1) // page for o, q in zip(old_lens, q_lens)) + 1
    tq = sum(q_lens)
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    bt = torch.randperm(nb * W, generator=g).to(torch.int32).reshape(nb, W)
    q = torch.randn(tq, heads, dim, generator=g).to(dtype)
    kn = torch.randn(tq, heads_kv, dim, generator=g).to(dtype)
    vn = torch.randn(tq, heads_kv, dim, generator=g).to(dtype)
    kp = torch.full((nb * W * page, heads_kv, dim), pool_fill).to(dtype)
    vp = torch.full((nb * W * page, heads_kv, dim), pool_fill).to(dtype)
    for b, n in enumerate(old_lens):
        rows = torch.from_numpy(O.physical_rows(bt[b].numpy(), n, page))
        kp[rows] = torch.randn(n, heads_kv, dim, generator=g).to(dtype)
        vp[rows] = torch.randn(n, heads_kv, dim, generator=g).to(dtype)
    cache = torch.tensor(old_lens, dtype=torch.int32)
    return q, kn, vn, kp, vp, cu, cache, bt


def _run(case, page, max_q, **kw):
    q, kn, vn, kp, vp, cu, cache, bt = (x.cuda() for x in case)
    o = _F().gqa_prefill_paged(q, kn, vn, kp, vp, cu, cache, bt, max_q, page_size=page, **kw)
    torch.cuda.synchronize()
    assert _F().prefill_status(q.device) == 0
    return o.cpu(), kp.cpu(), vp.cpu()


def _check(q_lens, old_lens, heads, heads_kv, dim, page, dtype, is_causal=True, softcap=None, **ckw):
    case = _case(q_lens, old_lens, heads, heads_kv, dim, page, dtype, **ckw)
    ref_o, ref_kp, ref_vp = O.prefill_paged_ref(*case, page, is_causal=is_causal, softcap=softcap)
    o, kp, vp = _run(case, page, max(q_lens), is_causal=is_causal, softcap=softcap or 0.0)
    torch.testing.assert_close(o.float(), ref_o.float(), **TOL[dtype])
    # the append is a copy: bit exact, and nothing else in the pool moves
    assert torch.equal(kp.view(torch.int16), ref_kp.view(torch.int16))
    assert torch.equal(vp.view(torch.int16), ref_vp.view(torch.int16))


@pytest.mark.parametrize("q_lens,old_lens,heads,heads_kv,is_causal,dtype", [
    ([64, 96], [80, 128], 8, 2, True, torch.float16),
    ([17, 33], [37, 100], 8, 2, True, torch.float16),
    ([1], [511], 8, 2, True, torch.float16),
    ([1, 17], [511, 37], 8, 2, True, torch.float16),
    ([64, 64], [64, 128], 8, 8, True, torch.float16),
    ([32, 64], [96, 160], 8, 1, True, torch.float16),
    ([64, 96], [80, 128], 8, 2, False, torch.float16),
    ([64, 96], [80, 128], 8, 2, True, torch.bfloat16),
])
def test_reference_cases_dim64(q_lens, old_lens, heads, heads_kv, is_causal, dtype):
    _check(q_lens, old_lens, heads, heads_kv, 64, 64, dtype, is_causal=is_causal, pages_per_req=8)


def _random_case(seed):
    import random
    rng = random.Random(4321 + seed)
    dim = rng.choice([64, 128, 128, 256])
    heads_kv = rng.choice([1, 2, 4])
    heads = heads_kv * rng.choice([1, 2, 4, 8])
    page = rng.choice([16, 32, 64, 128])
    nb = rng.choice([1, 2, 3, 5])
    q_lens = [rng.choice([1, 2, 63, 64, 65, 127, 128, 129, rng.randint(1, 300)]) for _ in range(nb)]
    old_lens = [rng.choice([0, 1, 63, 64, 65, page, rng.randint(0, 700)]) for _ in range(nb)]
    return dict(q_lens=q_lens, old_lens=old_lens, heads=heads, heads_kv=heads_kv, dim=dim, page=page,
                dtype=rng.choice([torch.float16, torch.bfloat16]), is_causal=rng.random() < 0.75,
                softcap=rng.choice([None, None, 20.0]), seed=seed)


@pytest.mark.parametrize("seed", range(24))
def test_random_paged_prefill_matches_the_oracle(seed):
    """Seeded random chunks over random caches (head dim 64 / 128 / 256, page 16 ... 128, ragged request and cache
    lengths around the 64-key and 128-row tile edges, requests without a cache, NaN in every pool row that holds
    no token): output against the oracle, appended rows bit for bit, nothing else in the pool touched."""
    c = _random_case(seed)
    _check(c["q_lens"], c["old_lens"], c["heads"], c["heads_kv"], c["dim"], c["page"], c["dtype"], is_causal=c["is_causal"],
           softcap=c["softcap"], seed=c["seed"], pool_fill=float("nan"))


@pytest.mark.parametrize("page", [16, 32, 64, 128, 256])
def test_page_sizes(page):
    _check([32, 64], [48, 80], 8, 2, 64, page, torch.float16, pages_per_req=16)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("dim", [64, 128])
def test_ragged_multi_tile(dim, dtype):
    # several 128-row tiles per request, empty cache, cache shorter than a tile, unaligned everything
    _check([300, 1, 129, 257], [0, 5, 1000, 333], 8, 2, dim, 16, dtype, seed=3)


def test_head_dim_256_with_partial_rope_like_the_qwen_workloads():
    # manifest workloads "qwen35-9b-prefill-paged-*": head dim 256, rotary_dim 64, page 64 (lengths scaled down)
    from tileops_b200.ops import GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp
    q_lens, old_lens, heads, heads_kv, dim, page, W_ = [130, 70, 257], [500, 64, 3], 8, 2, 256, 64, 16
    dtype = torch.float16
    q, kn, vn, kp, vp, cu, cache, bt = _case(q_lens, old_lens, heads, heads_kv, dim, page, dtype, seed=33,
                                             pages_per_req=W_)
    _check(q_lens, old_lens, heads, heads_kv, dim, page, dtype, seed=33, pages_per_req=W_)
    max_position = W_ * page
    op = GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp(
        batch=3, heads=heads, heads_kv=heads_kv, max_pages_per_req=W_, page_size=page, dim=dim, fuse_rope=True,
        max_position=max_position, rotary_dim=64)
    # the operator builds its tables on the device (as the reference does); device and host cos / sin may
    # differ in the last bit, so the oracle rotates with the operator's own tables
    cos, sin = (t.cpu() for t in op._get_rope_cos_sin(torch.device("cuda", 0), dtype))
    torch.testing.assert_close(cos.float(), O.rope_tables_ref(64, max_position, dtype=dtype)[0].float(), atol=2e-3, rtol=0)
    q_rot = O.rope_neox_packed_ref(q, cos, sin, cu, cache, 64)
    k_rot = O.rope_neox_packed_ref(kn, cos, sin, cu, cache, 64)
    ref_o, ref_kp, _ = O.prefill_paged_ref(q_rot, k_rot, vn, kp, vp, cu, cache, bt, page)
    kpd, vpd = kp.cuda(), vp.cuda()
    one = torch.ones(1, device="cuda")
    o = op(q.cuda(), kn.cuda(), vn.cuda(), kpd, vpd, one, one.clone(), cu.cuda(), cache.cuda(), bt.cuda(), max(q_lens))
    torch.testing.assert_close(o.cpu().float(), ref_o.float(), **TOL[dtype])
    assert torch.equal(kpd.cpu().view(torch.int16), ref_kp.view(torch.int16))


def test_softcap_and_noncausal_dim128():
    _check([200, 77], [130, 64], 16, 4, 128, 64, torch.bfloat16, softcap=30.0, seed=4)
    _check([200, 77], [130, 64], 16, 4, 128, 64, torch.bfloat16, is_causal=False, seed=5)


def test_unwritten_pool_memory_cannot_leak_into_the_result():
    # every pool row that holds no cached token is NaN: the rows behind a ragged last tile are
    # loaded with it and must not reach O
    case = _case([70, 33], [37, 100], 8, 2, 128, 16, torch.bfloat16, seed=6, pool_fill=float("nan"))
    ref_o, _, _ = O.prefill_paged_ref(*case, 16, is_causal=True)
    o, _, _ = _run(case, 16, 70)
    assert torch.isfinite(o.float()).all()
    torch.testing.assert_close(o.float(), ref_o.float(), **TOL[torch.bfloat16])


def test_golden_vectors():
    G = np.load(os.path.join(HERE, "golden", "gqa_golden.npz"))
    names = ["pp_q", "pp_k_new", "pp_v_new", "pp_k_pages", "pp_v_pages", "pp_cu", "pp_cache", "pp_bt"]
    case = [torch.from_numpy(G[n]) for n in names]
    page = int(G["pp_page"])
    # the fixture is D = 32; the kernel serves 64: zero-pad the head dim (scores and outputs are
    # unchanged by zero columns) and pass the fixture's scale
    def pad(x):
        return torch.cat([x, torch.zeros_like(x)], dim=-1).half()
    case[:5] = [pad(x) for x in case[:5]]
    o, kp, vp = _run(case, page, 33, sm_scale=32 ** -0.5)
    torch.testing.assert_close(o[..., :32].float(), torch.from_numpy(G["pp_o_causal"]), atol=5e-3, rtol=5e-3)
    assert torch.equal(kp[..., :32], torch.from_numpy(G["pp_k_pages_after"]).half())
    assert torch.equal(vp[..., :32], torch.from_numpy(G["pp_v_pages_after"]).half())
    o, _, _ = _run(case, page, 33, sm_scale=32 ** -0.5, is_causal=False)
    torch.testing.assert_close(o[..., :32].float(), torch.from_numpy(G["pp_o_full"]), atol=5e-3, rtol=5e-3)


def test_no_cache_is_packed_varlen_prefill():
    g = torch.Generator().manual_seed(9)
    q_lens = [5, 128, 200, 64]
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    q = torch.randn(sum(q_lens), 8, 128, generator=g).bfloat16()
    k = torch.randn(sum(q_lens), 2, 128, generator=g).bfloat16()
    v = torch.randn(sum(q_lens), 2, 128, generator=g).bfloat16()
    ref = O.prefill_packed_ref(q, k, v, cu, cu, is_causal=True)
    o = _F().gqa_prefill_paged(q.cuda(), k.cuda(), v.cuda(), None, None, cu.cuda(), None, None, 200)
    torch.testing.assert_close(o.cpu().float(), ref.float(), **TOL[torch.bfloat16])


def test_decode_reads_what_prefill_appended():
    # chunked prefill of one request in two chunks, then one decode step over the pages, equals the
    # oracle's attention over the whole sequence
    F = _F()
    g = torch.Generator().manual_seed(11)
    H, Hkv, D, page, W = 16, 4, 128, 64, 8
    n1, n2 = 200, 131
    bt = torch.randperm(W, generator=g).to(torch.int32).reshape(1, W).cuda()
    kp = torch.full((W * page, Hkv, D), float("nan")).bfloat16().cuda()
    vp = torch.full((W * page, Hkv, D), float("nan")).bfloat16().cuda()
    k = torch.randn(n1 + n2, Hkv, D, generator=g).bfloat16()
    v = torch.randn(n1 + n2, Hkv, D, generator=g).bfloat16()
    q = torch.randn(n1 + n2, H, D, generator=g).bfloat16()
    o1 = F.gqa_prefill_paged(q[:n1].cuda(), k[:n1].cuda(), v[:n1].cuda(), kp, vp,
                             torch.tensor([0, n1], dtype=torch.int32).cuda(),
                             torch.tensor([0], dtype=torch.int32).cuda(), bt, n1, page_size=page)
    o2 = F.gqa_prefill_paged(q[n1:].cuda(), k[n1:].cuda(), v[n1:].cuda(), kp, vp,
                             torch.tensor([0, n2], dtype=torch.int32).cuda(),
                             torch.tensor([n1], dtype=torch.int32).cuda(), bt, n2, page_size=page)
    ref = O.prefill_ref(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0), is_causal=True)[0]
    torch.testing.assert_close(torch.cat([o1, o2]).cpu().float(), ref.float(), **TOL[torch.bfloat16])
    qd = torch.randn(1, H, D, generator=g).bfloat16()
    od = F.gqa_decode(qd.cuda(), kp, vp, real_seqlen_kv=torch.tensor([n1 + n2], dtype=torch.int32).cuda(),
                      block_table=bt, page_size=page)
    refd = O.decode_ref(qd, k.unsqueeze(0), v.unsqueeze(0))
    torch.testing.assert_close(od.cpu().float(), refd.float(), **TOL[torch.bfloat16])


def test_llama8b_chunk_shape_property():
    # manifest workload "llama-8b-prefill-paged-b8-prefix4k-chunk512-p64" (without the fused RoPE):
    # full size on the GPU; checked on two requests by the oracle and on all by a chunk-invariance
    # property: splitting the chunk in two calls gives the same rows (bitwise for the first half).
    F = _F()
    g = torch.Generator().manual_seed(12)
    B, H, Hkv, D, page, W, old, n = 8, 32, 8, 128, 64, 72, 4096, 512
    bt = torch.randperm(B * W, generator=g).to(torch.int32).reshape(B, W)
    kp = torch.randn(B * W * page, Hkv, D, generator=g).half()
    vp = torch.randn(B * W * page, Hkv, D, generator=g).half()
    q = torch.randn(B * n, H, D, generator=g).half()
    kn = torch.randn(B * n, Hkv, D, generator=g).half()
    vn = torch.randn(B * n, Hkv, D, generator=g).half()
    cu = torch.arange(B + 1, dtype=torch.int32) * n
    cache = torch.full((B,), old, dtype=torch.int32)
    ref_o, ref_kp, _ = O.prefill_paged_ref(q[:2 * n], kn[:2 * n], vn[:2 * n], kp, vp, cu[:3], cache[:2], bt[:2], page)
    kpd, vpd = kp.cuda(), vp.cuda()
    o = F.gqa_prefill_paged(q.cuda(), kn.cuda(), vn.cuda(), kpd, vpd, cu.cuda(), cache.cuda(), bt.cuda(), n,
                            page_size=page)
    torch.testing.assert_close(o[:2 * n].cpu().float(), ref_o.float(), **TOL[torch.float16])
    rows = torch.from_numpy(O.physical_rows(bt[1].numpy(), old + n, page))
    assert torch.equal(kpd.cpu()[rows], ref_kp[rows])
    # first half of every chunk alone (cache unchanged by construction: same pages rewritten with the same rows)
    half = n // 2
    idx = (torch.arange(B)[:, None] * n + torch.arange(half)[None]).reshape(-1)
    cu2 = torch.arange(B + 1, dtype=torch.int32) * half
    o_half = F.gqa_prefill_paged(q[idx].cuda(), kn[idx].cuda(), vn[idx].cuda(), kpd, vpd, cu2.cuda(), cache.cuda(),
                                 bt.cuda(), half, page_size=page)
    assert torch.equal(o_half.cpu(), o.cpu()[idx])


# ---- through the operator classes (the reference's call shape) ------------------------------------

def test_paged_op_like_the_reference_test():
    from tileops_b200.ops import GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp
    q_lens, old_lens, heads, heads_kv, dim, page, W = [17, 33], [37, 100], 8, 2, 64, 64, 8
    for dtype in (torch.float16, torch.bfloat16):   # one instance serves both element types
        case = _case(q_lens, old_lens, heads, heads_kv, dim, page, dtype, pages_per_req=W, seed=20)
        ref_o, ref_kp, ref_vp = O.prefill_paged_ref(*case, page, is_causal=True)
        q, kn, vn, kp, vp, cu, cache, bt = (x.cuda() for x in case)
        op = GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp(
            batch=2, heads=heads, heads_kv=heads_kv, max_pages_per_req=W, page_size=page, dim=dim)
        one = torch.ones(1, device="cuda")
        o = op(q, kn, vn, kp, vp, one, one.clone(), cu, cache, bt, max(q_lens))
        assert isinstance(o, torch.Tensor) and o.shape == q.shape and o.dtype == dtype
        torch.testing.assert_close(o.cpu().float(), ref_o.float(), **TOL[dtype])
        assert torch.equal(kp.cpu().view(torch.int16), ref_kp.view(torch.int16))
        assert torch.equal(vp.cpu().view(torch.int16), ref_vp.view(torch.int16))
        with pytest.raises(ValueError, match="exceeds paged KV capacity"):
            op(q, kn, vn, kp, vp, one, one, cu, cache + 450, bt, max(q_lens))
        with pytest.raises(ValueError, match="block_table references page"):
            op(q, kn, vn, kp, vp, one, one, cu, cache, bt + 100, max(q_lens))
        with pytest.raises(ValueError, match="max_seqlen_q"):
            op(q, kn, vn, kp, vp, one, one, cu, cache, bt, 8)


@pytest.mark.parametrize("causal", [True, False])
def test_varlen_op_with_longer_kv(causal):
    from tileops_b200.ops import GroupedQueryAttentionPrefillFwdOp, GroupedQueryAttentionPrefillVarlenFwdOp
    g = torch.Generator().manual_seed(21)
    q_lens, kv_lens, H, Hkv, D = [24, 130, 1, 257], [50, 130, 300, 400], 8, 2, 128
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(np.cumsum(kv_lens)), dtype=torch.int32)
    q = torch.randn(sum(q_lens), H, D, generator=g).bfloat16()
    k = torch.randn(sum(kv_lens), Hkv, D, generator=g).bfloat16()
    v = torch.randn(sum(kv_lens), Hkv, D, generator=g).bfloat16()
    ref = O.prefill_packed_ref(q, k, v, cu_q, cu_k, is_causal=causal)
    op = GroupedQueryAttentionPrefillVarlenFwdOp(4, H, Hkv, D, max(q_lens), max(kv_lens), is_causal=causal,
                                                 validate_inputs=True)
    o = op(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda())
    torch.testing.assert_close(o.cpu().float(), ref.float(), **TOL[torch.bfloat16])
    flops, nbytes = op.eval_roofline()
    assert flops > 0 and nbytes > 0
    # the canonical packed op reaches the same kernel when the request is ragged
    op2 = GroupedQueryAttentionPrefillFwdOp(4, H, Hkv, D, max(q_lens), max(kv_lens), dtype=torch.bfloat16,
                                            is_causal=causal)
    ones = torch.ones(4, Hkv, device="cuda")
    o2 = op2(q.cuda(), k.cuda(), v.cuda(), cu_q.cuda(), cu_k.cuda(), ones, ones.clone(), ones.clone())
    assert torch.equal(o2, o)


# ---- RoPE ------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rotary_dim", [None, 32])
def test_rope_neox_packed_is_bit_exact(rotary_dim, dtype):
    g = torch.Generator().manual_seed(30)
    q_lens, old_lens, H, D = [48, 33, 1], [67, 100, 0], 8, 64
    cu = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    cache = torch.tensor(old_lens, dtype=torch.int32)
    x = torch.randn(sum(q_lens), H, D, generator=g).to(dtype)
    cos, sin = O.rope_tables_ref(rotary_dim or D, 200, dtype=dtype)
    y = _F().rope_neox_packed(x.cuda(), cos.cuda(), sin.cuda(), cu.cuda(), cache.cuda(), rotary_dim)
    ref = O.rope_neox_packed_ref(x, cos, sin, cu, cache, rotary_dim)
    assert torch.equal(y.cpu().view(torch.int16), ref.view(torch.int16))


def test_rope_golden_vectors():
    G = np.load(os.path.join(HERE, "golden", "gqa_golden.npz"))

    def h(name):
        return torch.from_numpy(G[name].view(np.int16)).view(torch.float16)
    cu = torch.tensor([0, 17, 50], dtype=torch.int32).cuda()
    cache = torch.tensor([37, 100], dtype=torch.int32).cuda()
    for name, rd in (("full", 32), ("partial", 16)):
        y = _F().rope_neox_packed(h("rope_x").cuda(), h("rope_cos_" + name).cuda(), h("rope_sin_" + name).cuda(),
                                  cu, cache, rd)
        assert torch.equal(y.cpu(), h("rope_y_" + name))


@pytest.mark.parametrize("rotary_dim,is_causal,softcap", [(None, True, None), (32, True, None), (32, False, None),
                                                          (32, True, 2.0)])
def test_paged_op_with_rope_like_the_reference_test(rotary_dim, is_causal, softcap):
    # tests/ops/attention/test_gqa_prefill_paged.py:476-590 of the reference: raw q / k_new go in; the result
    # equals attention over rotated q and keys, and the pages receive the rotated keys
    from tileops_b200.ops import GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp
    q_lens, old_lens, heads, heads_kv, dim, page, W = [48, 33], [67, 100], 8, 2, 64, 64, 8
    dtype = torch.float16
    max_position = max(o + n for o, n in zip(old_lens, q_lens)) + 1
    q, kn, vn, kp, vp, cu, cache, bt = _case(q_lens, old_lens, heads, heads_kv, dim, page, dtype, seed=31,
                                             pages_per_req=W)
    op = GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp(
        batch=2, heads=heads, heads_kv=heads_kv, max_pages_per_req=W, page_size=page, dim=dim, is_causal=is_causal,
        softcap=softcap, fuse_rope=True, max_position=max_position, rotary_dim=rotary_dim)
    cos, sin = (t.cpu() for t in op._get_rope_cos_sin(torch.device("cuda", 0), dtype))   # the operator's tables
    q_rot = O.rope_neox_packed_ref(q, cos, sin, cu, cache, rotary_dim)
    k_rot = O.rope_neox_packed_ref(kn, cos, sin, cu, cache, rotary_dim)
    ref_o, ref_kp, ref_vp = O.prefill_paged_ref(q_rot, k_rot, vn, kp, vp, cu, cache, bt, page, is_causal=is_causal,
                                                softcap=softcap)
    kpd, vpd = kp.cuda(), vp.cuda()
    one = torch.ones(1, device="cuda")
    o = op(q.cuda(), kn.cuda(), vn.cuda(), kpd, vpd, one, one.clone(), cu.cuda(), cache.cuda(), bt.cuda(), max(q_lens))
    torch.testing.assert_close(o.cpu().float(), ref_o.float(), atol=5e-3, rtol=1e-3)
    assert torch.equal(kpd.cpu().view(torch.int16), ref_kp.view(torch.int16))
    assert torch.equal(vpd.cpu().view(torch.int16), ref_vp.view(torch.int16))
    with pytest.raises(ValueError, match="exceeds RoPE max_position"):
        op(q.cuda(), kn.cuda(), vn.cuda(), kpd, vpd, one, one, cu.cuda(), cache.cuda() + 2, bt.cuda(), max(q_lens))


# ---- FP8-e4m3 cache with scalar scales ---------------------------------------------------------------

@pytest.mark.parametrize("is_causal,softcap,dtype,page,dim", [
    (True, None, torch.float16, 64, 64), (False, None, torch.float16, 64, 64), (True, 2.0, torch.float16, 64, 64),
    (True, None, torch.bfloat16, 64, 64), (True, None, torch.float16, 16, 64), (True, None, torch.float16, 128, 64),
    (True, None, torch.bfloat16, 64, 128),
])
def test_paged_op_with_fp8_cache_like_the_reference_test(is_causal, softcap, dtype, page, dim):
    # tests/ops/attention/test_gqa_prefill_paged.py:303-410 of the reference
    from tileops_b200.ops import GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp
    f8 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(40)
    q_lens, old_lens, heads, heads_kv, W = [33, 48], [67, 80], 8, 2, 8 * 64 // page
    cu = torch.tensor([0, 33, 81], dtype=torch.int32)
    cache = torch.tensor(old_lens, dtype=torch.int32)
    bt = torch.randperm(2 * W, generator=g).to(torch.int32).reshape(2, W)
    ks, vs = torch.tensor([0.02]), torch.tensor([0.025])
    q = torch.randn(81, heads, dim, generator=g).to(dtype)
    kn = (torch.randn(81, heads_kv, dim, generator=g) * 0.5).to(dtype)
    vn = (torch.randn(81, heads_kv, dim, generator=g) * 0.5).to(dtype)
    kp = torch.zeros(2 * W * page, heads_kv, dim, dtype=f8)
    vp = torch.zeros_like(kp)
    for b, n in enumerate(old_lens):
        rows = torch.from_numpy(O.physical_rows(bt[b].numpy(), n, page))
        kp[rows] = ((torch.randn(n, heads_kv, dim, generator=g) * 0.5).to(dtype).float() / ks[0]).to(f8)
        vp[rows] = ((torch.randn(n, heads_kv, dim, generator=g) * 0.5).to(dtype).float() / vs[0]).to(f8)
    ref_o, ref_kp, ref_vp = O.prefill_paged_fp8_cache_ref(q, kn, vn, kp, vp, ks, vs, cu, cache, bt, page,
                                                          is_causal=is_causal, softcap=softcap)
    op = GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp(
        batch=2, heads=heads, heads_kv=heads_kv, max_pages_per_req=W, page_size=page, dim=dim, is_causal=is_causal,
        cache_dtype=f8, softcap=softcap)
    kpd, vpd = kp.cuda(), vp.cuda()
    o = op(q.cuda(), kn.cuda(), vn.cuda(), kpd, vpd, ks.cuda(), vs.cuda(), cu.cuda(), cache.cuda(), bt.cuda(), 48)
    torch.testing.assert_close(o.cpu().float(), ref_o.float(), **TOL[dtype])
    # quantise-on-append is bit exact and nothing else in the pool moves
    assert torch.equal(kpd.cpu().view(torch.uint8), ref_kp.view(torch.uint8))
    assert torch.equal(vpd.cpu().view(torch.uint8), ref_vp.view(torch.uint8))
    with pytest.raises(ValueError, match="finite positive"):
        op(q.cuda(), kn.cuda(), vn.cuda(), kpd, vpd, ks.cuda() * 0, vs.cuda(), cu.cuda(), cache.cuda(), bt.cuda(), 48)


@pytest.mark.parametrize("dtype,page,is_causal,softcap,q_lens,old_lens", [
    (torch.float16, 64, True, None, [200, 130], [300, 1]),        # two row tiles, ragged last cached tile
    (torch.bfloat16, 16, True, None, [33, 48, 1], [67, 80, 0]),   # small pages; a request with no cache yet
    (torch.float16, 32, True, 2.0, [129, 5], [64, 127]),          # softcap; cache length exactly one tile / one short
    (torch.bfloat16, 128, False, None, [64, 64], [1000, 513]),    # many cached tiles, non-causal chunk
])
def test_fused_fp8_cache_prefill_at_head_dim_128(dtype, page, is_causal, softcap, q_lens, old_lens):
    """The one-launch path (``fused=True``: e4m3 pages read by TMA, expanded in shared memory by the converter
    warps, scalar scales folded into the softmax, chunk quantised on append) against the dequantise-then-attend
    oracle, against the three-launch path, and the pages bit for bit."""
    F = _F()
    f8 = torch.float8_e4m3fn
    g = torch.Generator().manual_seed(44)
    heads, heads_kv, dim = 8, 2, 128
    B = len(q_lens)
    W = -(-(max(o + n for o, n in zip(old_lens, q_lens))) // page) + 1
    cu = torch.zeros(B + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(q_lens).cumsum(0)
    total = int(cu[-1])
    cache = torch.tensor(old_lens, dtype=torch.int32)
    bt = torch.randperm(B * W, generator=g).to(torch.int32).reshape(B, W)
    ks, vs = torch.tensor([0.02]), torch.tensor([0.025])
    q = torch.randn(total, heads, dim, generator=g).to(dtype)
    kn = (torch.randn(total, heads_kv, dim, generator=g) * 0.5).to(dtype)
    vn = (torch.randn(total, heads_kv, dim, generator=g) * 0.5).to(dtype)
    # unwritten pool rows hold the e4m3 NaN code: a kernel that let one reach the MMA would show it
    kp = torch.full((B * W * page, heads_kv, dim), float("nan")).to(f8)
    vp = kp.clone()
    for b, n in enumerate(old_lens):
        if n:
            rows = torch.from_numpy(O.physical_rows(bt[b].numpy(), n, page))
            kp[rows] = ((torch.randn(n, heads_kv, dim, generator=g) * 0.5).to(dtype).float() / ks[0]).to(f8)
            vp[rows] = ((torch.randn(n, heads_kv, dim, generator=g) * 0.5).to(dtype).float() / vs[0]).to(f8)
    ref_o, ref_kp, ref_vp = O.prefill_paged_fp8_cache_ref(q, kn, vn, kp, vp, ks, vs, cu, cache, bt, page,
                                                          is_causal=is_causal, softcap=softcap)
    dev = [x.cuda() for x in (q, kn, vn)]
    meta = [x.cuda() for x in (ks, vs, cu, cache, bt)]
    outs = {}
    for fused in (True, False):
        kpd, vpd = kp.cuda(), vp.cuda()
        o = F.gqa_prefill_paged_fp8_cache(*dev, kpd, vpd, *meta, max(q_lens), page_size=page, is_causal=is_causal,
                                          softcap=softcap or 0.0, fused=fused)
        assert not torch.isnan(o).any()
        torch.testing.assert_close(o.cpu().float(), ref_o.float(), **TOL[dtype])
        live = ~torch.isnan(ref_kp.float())
        assert torch.equal(kpd.cpu().view(torch.uint8)[live], ref_kp.view(torch.uint8)[live])
        assert torch.equal(vpd.cpu().view(torch.uint8)[live], ref_vp.view(torch.uint8)[live])
        assert torch.equal(kpd.cpu().view(torch.uint8)[~live], kp.view(torch.uint8)[~live])      # nothing else moved
        outs[fused] = o
    torch.testing.assert_close(outs[True].float(), outs[False].float(), atol=4e-3, rtol=1e-2)
    # the same choice through the kernel class's config= (the tuning surface of the operator layer)
    from tileops_b200.kernels.gqa_prefill import GQAPrefillPagedFp8CacheSm100Kernel
    kern = GQAPrefillPagedFp8CacheSm100Kernel(B, heads, heads_kv, W, page, dim, is_causal, dtype, softcap=softcap or 0.0,
                                              config={"fused": True})
    assert kern.config["fused"] is True
    o2 = kern.forward(*dev, kp.cuda(), vp.cuda(), *meta, max(q_lens))
    assert torch.equal(o2, outs[True])


def test_fp8_cache_golden_vectors():
    G = np.load(os.path.join(HERE, "golden", "gqa_golden.npz"))

    def h(name):
        return torch.from_numpy(G[name].view(np.int16)).view(torch.float16)

    def f8(name):
        return torch.from_numpy(G[name]).view(torch.float8_e4m3fn)

    def pad(x):   # D = 32 fixtures, the kernel serves 64: zero columns (zero is exact in e4m3 too)
        return torch.cat([x, torch.zeros_like(x)], dim=-1).cuda()
    kp, vp = pad(f8("p8_k_pages")), pad(f8("p8_v_pages"))
    args = (pad(h("p8_q")), pad(h("p8_k_new")), pad(h("p8_v_new")), kp, vp, torch.from_numpy(G["p8_k_scale"]).cuda(),
            torch.from_numpy(G["p8_v_scale"]).cuda(), torch.from_numpy(G["p8_cu"]).cuda(),
            torch.from_numpy(G["p8_cache"]).cuda(), torch.from_numpy(G["p8_bt"]).cuda())
    page = int(G["p8_page"])
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")          # the call must not read anything back from the device
    try:
        o = _F().gqa_prefill_paged_fp8_cache(*args, 48, page_size=page, sm_scale=32 ** -0.5)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.testing.assert_close(o[..., :32].cpu().float(), h("p8_o").float(), atol=5e-3, rtol=1e-2)
    assert torch.equal(kp[..., :32].cpu().view(torch.uint8), f8("p8_k_pages_after").view(torch.uint8))
    assert torch.equal(vp[..., :32].cpu().view(torch.uint8), f8("p8_v_pages_after").view(torch.uint8))


def test_last_cached_tile_never_reads_behind_the_block_table_row():
    """5 pages of 16 tokens, 79 cached + 1 new: the last 64-key tile of the cache covers tokens 64..127,
    past the 80 the table describes.  The lookup for the tile's tail must stay inside the request's row
    (here the LAST row of the table, which ends its allocation); the result must still match."""
    for heads_kv in (2, 8):
        _check([1, 1], [40, 79], 8, heads_kv, 64, 16, torch.float16, pages_per_req=5, pool_fill=float("nan"))
