"""Guard-band tests: every buffer a kernel writes (o, LSE, the decode workspace, the pages an append may touch)
sits between two bands of a known byte pattern, and the bands must come back untouched.

The reference has no analogue (TileLang bounds its own buffers); these tests stand in for a debug build with
bounds assertions: the shapes are ragged on purpose (tail pages, sequence lengths that are no multiple of any
tile, row counts that are no multiple of the 128-row q tile), which is where an off-by-one store would land.
"""

import pytest
import torch

from tileops_b200 import _native as N
from tileops_b200 import functional as F
from tileops_b200 import workloads as W

pytestmark = pytest.mark.gpu

GUARD = 4096          # bytes on each side
PATTERN = 0xA5


def guarded(nbytes: int, device, fill: int = 0):
    """(whole buffer, the guarded middle as uint8) with the middle 256-byte aligned."""
    assert GUARD % 256 == 0
    body = -(-nbytes // 256) * 256
    whole = torch.full((GUARD + body + GUARD,), PATTERN, dtype=torch.uint8, device=device)
    mid = whole[GUARD:GUARD + nbytes]
    mid.fill_(fill)
    whole[GUARD + nbytes:GUARD + body].fill_(PATTERN)
    return whole, mid


def assert_guards(whole: torch.Tensor, nbytes: int, what: str):
    lo, hi = whole[:GUARD], whole[GUARD + nbytes:]
    assert bool((lo == PATTERN).all()), f"{what}: bytes before the buffer were written"
    assert bool((hi == PATTERN).all()), f"{what}: bytes behind the buffer were written"


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("config", [None, {"tma": False}])
def test_decode_writes_stay_inside_o_lse_and_workspace(monkeypatch, fp8, config):
    dev = torch.device("cuda")
    B, H, Hkv, D, page = 7, 32, 8, 128, 64
    lens = [1, 63, 64, 65, 1000, 4097, 0]
    inp = W.make_paged_decode(41, B, H, Hkv, D, page, lens=lens, fp8_cache=fp8, device=dev, tail_fill=float("nan"))
    o_whole, o_mid = guarded(B * H * D * 2, dev)
    l_whole, l_mid = guarded(B * H * 4, dev)
    need = N.lib().tb200_gqa_decode_workspace_bytes(B, H, Hkv, D)
    w_whole, w_mid = guarded(need, dev)
    monkeypatch.setattr(F, "_decode_workspace", lambda *a, **k: w_mid)
    out = o_mid.view(torch.bfloat16).view(B, H, D)
    lse = l_mid.view(torch.float32).view(B, H)
    kw = dict(k_scale=inp.k_scale, v_scale=inp.v_scale) if fp8 else {}
    for _ in range(3):     # the counters of the workspace are reused from call to call
        F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table,
                     page_size=page, out=out, lse_out=lse, config=config, **kw)
    torch.cuda.synchronize()
    assert_guards(o_whole, B * H * D * 2, "o")
    assert_guards(l_whole, B * H * 4, "lse")
    assert_guards(w_whole, need, "workspace")
    ref = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table,
                       page_size=page, config=config, **kw)
    assert torch.equal(out[:6], ref[:6])
    assert bool(torch.isfinite(out[:6].float()).all())


@pytest.mark.parametrize("seq_q,seq_kv", [(1, 1), (127, 127), (129, 300), (333, 333)])
def test_dense_prefill_writes_stay_inside_o_and_lse(seq_q, seq_kv):
    dev = torch.device("cuda")
    B, H, Hkv, D = 2, 8, 2, 128
    q, k, v = W.make_prefill(42, B, seq_q, seq_kv, H, Hkv, D, torch.bfloat16, dev)
    o_whole, o_mid = guarded(q.numel() * 2, dev)
    l_whole, l_mid = guarded(B * H * seq_q * 4, dev)
    need = N.lib().tb200_gqa_prefill_workspace_bytes(B, H, Hkv, seq_q, seq_kv, D)
    ws = F._prefill_status(dev, need)
    with torch.cuda.device(dev):
        st = N.lib().tb200_gqa_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), o_mid.data_ptr(), l_mid.data_ptr(),
                                       N.dtype_code(q.dtype), B, seq_q, seq_kv, H, Hkv, D, 1, float(D ** -0.5), 0.0,
                                       -1, -1, 0, N.ptr(ws), need, N.current_stream(dev))
    N.check(st, "tb200_gqa_prefill")
    torch.cuda.synchronize()
    assert_guards(o_whole, q.numel() * 2, "o")
    assert_guards(l_whole, B * H * seq_q * 4, "lse")
    ref, ref_lse = F.gqa_prefill(q, k, v, is_causal=True, return_lse=True)
    assert torch.equal(o_mid.view(torch.bfloat16).view_as(ref), ref)
    assert torch.equal(l_mid.view(torch.float32).view_as(ref_lse), ref_lse)


def test_paged_prefill_append_touches_only_the_new_rows():
    dev = torch.device("cuda")
    H, Hkv, D, page, Wp = 8, 2, 128, 16, 24
    new, old = [5, 130, 17], [3, 100, 0]
    args = list(W.make_paged_prefill(43, new, old, H, Hkv, D, page, Wp, torch.bfloat16, dev))
    q, k_new, v_new, k_pages, v_pages, _, _, cu_q, cache_lens, bt, _ = args
    rows = k_pages.shape[0]
    row_bytes = Hkv * D * 2
    kw, km = guarded(rows * row_bytes, dev)
    vw, vm = guarded(rows * row_bytes, dev)
    km.copy_(k_pages.view(torch.uint8).view(-1))
    vm.copy_(v_pages.view(torch.uint8).view(-1))
    kp = km.view(torch.bfloat16).view(rows, Hkv, D)
    vp = vm.view(torch.bfloat16).view(rows, Hkv, D)
    before_k, before_v = kp.clone(), vp.clone()
    F.gqa_prefill_paged(q, k_new, v_new, kp, vp, cu_q, cache_lens, bt, max(new), page_size=page)
    torch.cuda.synchronize()
    assert_guards(kw, rows * row_bytes, "k_pages")
    assert_guards(vw, rows * row_bytes, "v_pages")
    # exactly the rows of the new tokens changed, and they hold the new tokens
    touched = torch.zeros(rows, dtype=torch.bool, device=dev)
    off = 0
    for b, (n, o) in enumerate(zip(new, old)):
        pos = torch.arange(o, o + n, device=dev)
        r = bt[b, pos // page].long() * page + pos % page
        touched[r] = True
        assert torch.equal(kp[r], k_new[off:off + n])
        assert torch.equal(vp[r], v_new[off:off + n])
        off += n
    assert torch.equal(kp[~touched], before_k[~touched])
    assert torch.equal(vp[~touched], before_v[~touched])
