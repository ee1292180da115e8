"""GPU parity tests of the tcgen05 prefill kernel: op -> kernel class -> C ABI -> CUDA against the
CPU oracle (fp32 materialised reference of tests/ops/attention/test_gqa.py:109-139 in
tile-ai/TileOPs).  Tolerance: 2e-2 abs / 1e-2 rel; LSE (log2 domain) 2e-3 abs."""

import numpy as np
import pytest
import torch

from oracle import gqa_oracle as O
from tileops_b200 import functional as F
from tileops_b200 import workloads as W
from tileops_b200.ops import GroupedQueryAttentionFwdOp, GroupedQueryAttentionPrefillFwdOp

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2


def close(got, want, atol=ATOL, rtol=RTOL):
    got, want = got.float().cpu(), want.float().cpu()
    assert not torch.isnan(got).any(), "NaN in kernel output"
    torch.testing.assert_close(got, want, atol=atol, rtol=rtol)


def packed_inputs(q, k, v):
    B, Sq, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    cu_q = torch.arange(B + 1, device=q.device, dtype=torch.int32) * Sq
    cu_k = torch.arange(B + 1, device=q.device, dtype=torch.int32) * Skv
    ones = torch.ones(B, Hkv, device=q.device, dtype=torch.float32)
    return (q.reshape(B * Sq, H, D), k.reshape(B * Skv, Hkv, D), v.reshape(B * Skv, Hkv, D), cu_q, cu_k,
            ones, ones.clone(), ones.clone())


@pytest.mark.parametrize("B,S,H,Hkv,causal,dtype", [
    (1, 128, 2, 1, True, torch.bfloat16),
    (1, 128, 2, 1, False, torch.bfloat16),
    (1, 256, 8, 2, True, torch.bfloat16),
    (2, 512, 8, 2, True, torch.float16),
    (1, 1024, 8, 4, False, torch.float16),
    (2, 384, 4, 4, True, torch.bfloat16),
    (1, 200, 4, 2, True, torch.bfloat16),       # ragged last tile in q and kv
    (1, 77, 2, 2, False, torch.float16),
    (1, 2048, 32, 8, True, torch.bfloat16),
])
def test_fwd_op_matches_oracle(B, S, H, Hkv, causal, dtype):
    q, k, v = W.make_prefill(41, B, S, S, H, Hkv, 128, dtype, "cuda")
    op = GroupedQueryAttentionFwdOp(B, H, Hkv, S, 128, is_causal=causal)
    o, lse = op(q, k, v, return_lse=True)
    assert o.shape == q.shape and o.dtype == dtype and lse.shape == (B, H, S)
    ro, rl = O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), causal, return_lse=True)
    close(o, ro)
    torch.testing.assert_close(lse.cpu(), rl, atol=2e-3, rtol=1e-3)
    assert F.prefill_status("cuda:0") == 0
    assert op.eval_roofline()[0] == (4 * B * H * S * S * 128) // (2 if causal else 1)


@pytest.mark.parametrize("B,Sq,Skv,H,Hkv,causal,dtype", [
    (2, 256, 256, 8, 2, True, torch.float16),
    (1, 200, 333, 4, 4, True, torch.bfloat16),
    (1, 1024, 1024, 8, 1, False, torch.bfloat16),
    (1, 77, 77, 2, 1, True, torch.float16),
])
def test_head_dim_64(B, Sq, Skv, H, Hkv, causal, dtype):
    q, k, v = W.make_prefill(45, B, Sq, Skv, H, Hkv, 64, dtype, "cuda")
    o, lse = F.gqa_prefill(q, k, v, is_causal=causal, return_lse=True)
    ro, rl = O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), causal, return_lse=True)
    close(o, ro)
    torch.testing.assert_close(lse.cpu(), rl, atol=2e-3, rtol=1e-3)
    assert F.prefill_status("cuda:0") == 0


@pytest.mark.parametrize("B,Sq,Skv,H,Hkv,causal,dtype", [
    (1, 256, 256, 4, 1, True, torch.float16),
    (2, 200, 333, 4, 2, True, torch.bfloat16),
    (1, 640, 640, 8, 2, False, torch.bfloat16),
    (1, 1024, 1024, 8, 2, True, torch.bfloat16),
])
def test_head_dim_256(B, Sq, Skv, H, Hkv, causal, dtype):
    q, k, v = W.make_prefill(46, B, Sq, Skv, H, Hkv, 256, dtype, "cuda")
    o, lse = F.gqa_prefill(q, k, v, is_causal=causal, return_lse=True)
    ro, rl = O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), causal, return_lse=True)
    close(o, ro)
    torch.testing.assert_close(lse.cpu(), rl, atol=2e-3, rtol=1e-3)
    assert F.prefill_status("cuda:0") == 0


@pytest.mark.parametrize("Sq,Skv,causal", [(128, 256, True), (512, 4096, True), (96, 150, True),
                                           (150, 406, True), (256, 128, False), (64, 1000, False)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_packed_prefill_op_q_shorter_than_kv(Sq, Skv, causal, dtype):
    B, H, Hkv = 2, 8, 2
    q, k, v = W.make_prefill(42, B, Sq, Skv, H, Hkv, 128, dtype, "cuda")
    op = GroupedQueryAttentionPrefillFwdOp(B, H, Hkv, 128, Sq, Skv, dtype=dtype, is_causal=causal)
    o = op(*packed_inputs(q, k, v)).view(B, Sq, H, 128)
    close(o, O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), causal))
    flops, nbytes = op.eval_roofline()
    assert flops > 0 and nbytes > 0


def test_bottom_right_mask_known_answer():
    # tests/ops/attention/test_gqa.py:417-443 in the reference (head dim 128 here)
    B, Sq, Skv, H, Hkv, D = 1, 128, 256, 4, 2, 128
    q = torch.zeros(B, Sq, H, D, device="cuda", dtype=torch.float16)
    k = torch.zeros(B, Skv, Hkv, D, device="cuda", dtype=torch.float16)
    v = torch.zeros(B, Skv, Hkv, D, device="cuda", dtype=torch.float16)
    q[..., 0] = 1; k[..., 0] = 1
    v[:, :128, :, 0] = 1; v[:, 128:, :, 0] = 100
    op = GroupedQueryAttentionPrefillFwdOp(B, H, Hkv, D, Sq, Skv, dtype=torch.float16, is_causal=True)
    o = op(*packed_inputs(q, k, v)).view(B, Sq, H, D)
    assert o[0, 0, 0, 0] < 2 and o[0, -1, 0, 0] > 40
    close(o, O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), True))


@pytest.mark.parametrize("sm_scale,softcap", [(0.125, None), (None, 2.0), (0.05, 50.0)])
def test_prefill_scale_and_softcap(sm_scale, softcap):
    B, S, H, Hkv = 1, 300, 4, 2
    q, k, v = W.make_prefill(43, B, S, S, H, Hkv, 128, torch.bfloat16, "cuda")
    op = GroupedQueryAttentionFwdOp(B, H, Hkv, S, 128, is_causal=True, sm_scale=sm_scale, softcap=softcap)
    close(op(q, k, v), O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), True, sm_scale, softcap))


def test_causal_with_more_queries_than_keys_gives_zero_rows():
    # bottom-right alignment: the first Sq - Skv query rows see no key at all
    B, Sq, Skv, H, Hkv = 1, 384, 128, 2, 1
    q, k, v = W.make_prefill(44, B, Sq, Skv, H, Hkv, 128, torch.bfloat16, "cuda")
    o, lse = F.gqa_prefill(q, k, v, is_causal=True, return_lse=True)
    assert torch.all(o[:, :Sq - Skv] == 0) and torch.all(torch.isinf(lse[..., :Sq - Skv]))
    ro = O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), True)
    close(o[:, Sq - Skv:], ro[:, Sq - Skv:])


def test_golden_prefill_fixture_head_dim_128_embedding():
    """The committed reference outputs have head dim 32; embed them in dim 128 (zero padding
    leaves q.k unchanged when sm_scale is fixed to 32**-0.5) and compare with the reference's
    own fp32 outputs."""
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "gqa_golden.npz"))
    q, k, v = (torch.from_numpy(G[n]) for n in ("pre_q", "pre_k", "pre_v"))
    pad = lambda t: torch.nn.functional.pad(t, (0, 96)).cuda().bfloat16()  # noqa: E731
    o = F.gqa_prefill(pad(q), pad(k), pad(v), is_causal=True, sm_scale=32 ** -0.5)
    close(o[..., :32], torch.from_numpy(G["pre_o_causal"]))
    o = F.gqa_prefill(pad(q), pad(k), pad(v), is_causal=False, sm_scale=32 ** -0.5)
    close(o[..., :32], torch.from_numpy(G["pre_o_full"]))


def test_config2_rows_against_oracle_and_causal_prefix_property():
    """The causal prefill workload (4 x 4096, 32/8 heads) at full size.  (a) one (batch, KV head) slice against the oracle;
    (b) causality: the first 1024 rows of the 4096-token result equal a 1024-token prefill."""
    B, S, H, Hkv, D = 4, 4096, 32, 8, 128
    q, k, v = W.make_prefill(2, B, S, S, H, Hkv, D, torch.bfloat16, "cuda")
    op = GroupedQueryAttentionFwdOp(B, H, Hkv, S, D, is_causal=True)
    o, lse = op(q, k, v, return_lse=True)
    b, hk = 3, 5
    ro, rl = O.prefill_ref(q[b:b + 1, :, 4 * hk:4 * hk + 4].cpu(), k[b:b + 1, :, hk:hk + 1].cpu(),
                           v[b:b + 1, :, hk:hk + 1].cpu(), True, return_lse=True)
    close(o[b:b + 1, :, 4 * hk:4 * hk + 4], ro)
    torch.testing.assert_close(lse[b:b + 1, 4 * hk:4 * hk + 4].cpu(), rl, atol=2e-3, rtol=1e-3)
    o1 = F.gqa_prefill(q[:, :1024].contiguous(), k[:, :1024].contiguous(), v[:, :1024].contiguous(), is_causal=True)
    assert torch.equal(o1, o[:, :1024])
    assert F.prefill_status("cuda:0") == 0


@pytest.mark.parametrize("B,Sq,Skv,H,Hkv,causal,wl,wr,softcap,dtype", [
    (1, 1024, 1024, 8, 2, True, -1, -1, 0.0, torch.bfloat16),
    (2, 640, 640, 4, 4, True, -1, -1, 0.0, torch.float16),        # odd number of row tiles: a pair with one tile
    (1, 300, 777, 4, 2, True, -1, -1, 0.0, torch.bfloat16),       # Sq < Skv, ragged tiles on both sides
    (1, 777, 300, 4, 2, True, -1, -1, 0.0, torch.bfloat16),       # Sq > Skv: leading rows see no key
    (1, 512, 512, 4, 1, False, -1, -1, 0.0, torch.bfloat16),
    (1, 1024, 1024, 4, 2, True, 200, -1, 0.0, torch.bfloat16),    # causal sliding window: the tiles of a pair start at different keys
    (1, 900, 900, 4, 2, False, 100, 60, 0.0, torch.float16),
    (1, 512, 512, 4, 2, True, -1, -1, 30.0, torch.bfloat16),
])
def test_two_tile_and_one_tile_kernels_agree_with_the_oracle(B, Sq, Skv, H, Hkv, causal, wl, wr, softcap, dtype):
    """Head dim 128 is served by two kernels (two Q tiles per CTA in ping-pong with 128-key tiles; one Q
    tile per CTA with 64-key tiles); both against the oracle, LSE included."""
    q, k, v = W.make_prefill(44, B, Sq, Skv, H, Hkv, 128, dtype, "cuda")
    ro, rl = O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), causal, softcap=softcap or None, return_lse=True,
                           window_left=wl, window_right=wr)
    outs = []
    for tiles in (2, 1):
        o, lse = F.gqa_prefill(q, k, v, is_causal=causal, softcap=softcap, return_lse=True, window_size_left=wl,
                               window_size_right=wr, config={"tiles_per_cta": tiles})
        assert F.prefill_status() == 0
        assert not torch.isnan(o).any()
        close(o, ro)
        fin = torch.isfinite(rl)
        assert torch.equal(fin, torch.isfinite(lse.cpu()))
        torch.testing.assert_close(lse.cpu()[fin], rl[fin], atol=2e-3, rtol=1e-3)
        outs.append((o, lse))
    torch.testing.assert_close(outs[0][0].float(), outs[1][0].float(), atol=1e-2, rtol=1e-2)
    fin = torch.isfinite(outs[1][1])
    assert torch.equal(fin, torch.isfinite(outs[0][1]))
    torch.testing.assert_close(outs[0][1][fin], outs[1][1][fin], atol=2e-3, rtol=1e-3)


def test_mma_issue_probe_reports_the_floor_the_kernels_are_designed_around():
    """One tcgen05.mma (M = 128, K = 16) never costs less than its arithmetic (N / 2 clocks) and, on B200, not
    less than ~90 clocks whatever N is."""
    for n in (64, 128, 256):
        issued, done = F.mma_issue_probe(n, a_in_tmem=(n == 128))
        assert n / 2 <= done < 1000 and issued <= done + 1, (n, issued, done)


def test_a_timed_out_prefill_surfaces_at_the_next_call():
    """The status word of the prefill kernels is sticky (launches after a wait that ran out return with their
    outputs unwritten).  The host keeps a pinned mirror of it: the call after the failure raises and clears it.
    The failure is made on the host here - the word is set by hand, no device-side wait runs out."""
    from tileops_b200._native import NativeLibraryError
    q, k, v = W.make_prefill(45, 1, 128, 128, 2, 1, 128, torch.bfloat16, "cuda")
    F.gqa_prefill(q, k, v)                                    # creates the status word and its mirror
    torch.cuda.synchronize()
    ws = F._WORKSPACES[(q.device, "prefill_status")]
    ws[:4].view(torch.int32).fill_(302)                       # what a kernel leaves when a wait gives up
    F.gqa_prefill(q, k, v)                                    # returns at once on the device; mirrors the word
    torch.cuda.synchronize()
    with pytest.raises(NativeLibraryError, match="code 302"):
        F.gqa_prefill(q, k, v)
    torch.cuda.synchronize()
    assert F.prefill_status() == 0                            # cleared: the next call works again
    close(F.gqa_prefill(q, k, v), O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), True))


def _random_dense_case(seed):
    import random
    rng = random.Random(977 + seed)
    dim = rng.choice([64, 128, 128, 256])
    heads_kv = rng.choice([1, 2, 4])
    heads = heads_kv * rng.choice([1, 2, 4, 8])
    batch = rng.choice([1, 2, 3])
    sq = rng.choice([1, 63, 64, 127, 128, 129, 200, rng.randint(1, 400)])
    skv = sq + rng.choice([0, 0, 1, 64, rng.randint(0, 500)])       # bottom-right aligned when longer
    mode = rng.choice(["causal", "causal", "full", "window"])
    return dict(dim=dim, heads=heads, heads_kv=heads_kv, batch=batch, sq=sq, skv=skv, mode=mode,
                wl=rng.choice([0, 7, 64, 200]), wr=rng.choice([-1, 0, 5]), softcap=rng.choice([None, None, 25.0]),
                dtype=rng.choice([torch.float16, torch.bfloat16]))


@pytest.mark.parametrize("seed", range(24))
def test_random_dense_prefill_matches_the_oracle(seed):
    """Seeded random dense problems: head dim 64 / 128 / 256, sequence lengths around the 128-row and 64-key tile
    edges, K/V longer than Q (bottom-right aligned mask), causal / full / sliding window, softcap; output and
    log2-domain LSE against the oracle."""
    from tileops_b200 import functional as F
    c = _random_dense_case(seed)
    q, k, v = W.make_prefill(300 + seed, c["batch"], c["sq"], c["skv"], c["heads"], c["heads_kv"], c["dim"], c["dtype"], "cuda")
    kw = dict(is_causal=c["mode"] == "causal", softcap=c["softcap"] or 0.0)
    okw = dict(is_causal=c["mode"] == "causal", softcap=c["softcap"])
    if c["mode"] == "window":
        kw.update(window_size_left=c["wl"], window_size_right=c["wr"])
        okw.update(window_left=c["wl"], window_right=c["wr"])
    o, lse = F.gqa_prefill(q, k, v, return_lse=True, **kw)
    want, want_lse = O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), return_lse=True, **okw)
    assert not torch.isnan(o).any(), c
    tol = dict(atol=5e-3, rtol=1e-2) if c["dtype"] == torch.float16 else dict(atol=2e-2, rtol=1e-2)
    finite = torch.isfinite(want_lse)                    # [B, H, Sq]; a row that sees no key: zeros, LSE -inf
    rows = finite.transpose(1, 2)                        # [B, Sq, H]
    torch.testing.assert_close(o.cpu().float()[rows], want.float()[rows], **tol)
    assert torch.count_nonzero(o.cpu()[~rows]) == 0
    torch.testing.assert_close(lse.cpu()[finite], want_lse[finite], atol=2e-3, rtol=1e-3)
    assert torch.isinf(lse.cpu()[~finite]).all()
