"""`tb200_gqa_decode_noalloc`: the decode entry point for hosts that may not allocate device memory
(a serving runtime that owns the whole device through its own pool and forbids cudaMalloc after
start-up, or a plugin that must not bypass its host framework's allocator).  Its split-KV scratch is
a fixed array inside the library instead of a caller workspace.

Called here through the C ABI with raw pointers, and compared with the ordinary entry point
(`tb200_gqa_decode`, reached through `tileops_b200.functional.gqa_decode`) on the same inputs, on two
calls in a row and then on a different shape, which moves the counters inside the shared array.
The file sorts last on purpose: a failure here must not hide any other test."""

import pytest
import torch

from tileops_b200 import _native as N
from tileops_b200 import functional as F
from tileops_b200 import workloads as W

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2          # the tolerance of the other decode tests
MAX_SCRATCH = 24 << 20           # TB200_DECODE_STATIC_SCRATCH_BYTES


def decode_noalloc(inp, out):
    q, k = inp.q, inp.k
    B, H, D = q.shape
    fp8 = inp.k_scale is not None
    with torch.cuda.device(q.device):
        return N.lib().tb200_gqa_decode_noalloc(
            q.data_ptr(), k.data_ptr(), inp.v.data_ptr(), out.data_ptr(), None,
            inp.real_seqlen_kv.data_ptr(), 0, inp.block_table.data_ptr(), inp.block_table.shape[1],
            inp.k_scale.data_ptr() if fp8 else None, inp.v_scale.data_ptr() if fp8 else None,
            N.dtype_code(q.dtype), N.dtype_code(k.dtype), N.dtype_code(out.dtype),
            B, H, k.shape[1], D, inp.page_size, k.stride(0), k.stride(1), 0,
            D ** -0.5, 0.0, torch.cuda.current_stream(q.device).cuda_stream)


def reference(inp):
    kw = dict(k_scale=inp.k_scale, v_scale=inp.v_scale) if inp.k_scale is not None else {}
    return F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table,
                        page_size=inp.page_size, **kw)


def test_noalloc_entry_point_matches_the_workspace_entry_point_twice_in_a_row():
    inp = W.make_paged_decode(51, 8, 32, 8, 128, 64, len_range=(100, 6000), device="cuda")   # split-KV runs
    want = reference(inp)
    for call in range(2):
        out = torch.full_like(want, float("nan"))
        assert decode_noalloc(inp, out) == 0, N.lib().tb200_last_error()
        torch.cuda.synchronize()
        torch.testing.assert_close(out.float(), want.float(), atol=ATOL, rtol=RTOL)
        inp.q.mul_(-0.5)                     # new data for the second call, same scratch
        want = reference(inp)
    # another shape: its counters sit where the previous shape kept partial results
    inp2 = W.make_paged_decode(52, 3, 64, 8, 128, 64, lens=[4096, 1, 700], fp8_cache=True, device="cuda")
    out2 = torch.full((3, 64, 128), float("nan"), device="cuda", dtype=torch.bfloat16)
    assert decode_noalloc(inp2, out2) == 0, N.lib().tb200_last_error()
    torch.testing.assert_close(out2.float(), reference(inp2).float(), atol=ATOL, rtol=RTOL)
    out = torch.full_like(want, float("nan"))
    assert decode_noalloc(inp, out) == 0
    torch.testing.assert_close(out.float(), want.float(), atol=ATOL, rtol=RTOL)


def test_noalloc_entry_point_refuses_problems_beyond_its_scratch():
    lib = N.lib()
    B, H, Hkv, D = 2048, 128, 8, 128
    assert lib.tb200_gqa_decode_workspace_bytes(B, H, Hkv, D) > MAX_SCRATCH
    t = torch.zeros(16, device="cuda")
    p = t.data_ptr()
    st = lib.tb200_gqa_decode_noalloc(p, p, p, p, None, None, 1, p, 1, None, None, 1, 1, 1,
                                      B, H, Hkv, D, 64, 1024, 128, 0, 1.0, 0.0, None)
    assert st == 3
    msg = lib.tb200_last_error().decode()
    assert "built-in scratch holds" in msg and str(MAX_SCRATCH) in msg
