"""The ``tileops.backends`` plugin target "b200" end to end on a GPU: with the plugin registered, the
operators settle on the target by device detection and run through its builders."""

import numpy as np
import pytest
import torch

from oracle import gqa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture
def b200_target():
    from tileops_b200 import backend, plugin
    from tileops_b200.backend import registry
    state = registry.snapshot()
    plugin.register(backend)
    yield plugin.TARGET
    registry.restore(state)


def test_ops_settle_on_the_plugin_target_and_match_the_oracle(b200_target):
    from tileops_b200 import workloads as W
    from tileops_b200.ops import (GroupedQueryAttentionDecodePagedWithKVCacheFwdOp, GroupedQueryAttentionFwdOp,
                                  GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp)
    inp = W.make_paged_decode(31, 4, 16, 4, 128, 64, len_range=(100, 900), device="cuda")
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(4, 16, 4, inp.k.shape[0], 128, 64)
    o = op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    assert op._settled_target == b200_target
    ref = O.paged_decode_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv.cpu(), inp.block_table.cpu(), 64)
    torch.testing.assert_close(o.cpu().float(), ref.float(), atol=2e-2, rtol=1e-2)

    q, k, v = W.make_prefill(32, 2, 256, 256, 8, 2, 128, torch.bfloat16, "cuda")
    fwd = GroupedQueryAttentionFwdOp(2, 8, 2, 256, 128, is_causal=True)
    o = fwd(q, k, v)
    assert fwd._settled_target == b200_target
    torch.testing.assert_close(o.cpu().float(), O.prefill_ref(q.cpu(), k.cpu(), v.cpu(), True).float(),
                               atol=2e-2, rtol=1e-2)

    args = W.make_paged_prefill(33, [70, 200], [130, 64], 8, 2, 128, 64, 8, torch.float16, "cuda")
    pre = GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp(2, 8, 2, 8, 64, 128)
    cpu = [a.cpu() if isinstance(a, torch.Tensor) else a for a in args]
    ref_o, ref_kp, _ = O.prefill_paged_ref(cpu[0], cpu[1], cpu[2], cpu[3], cpu[4], cpu[7], cpu[8], cpu[9], 64)
    o = pre(*args)
    assert pre._settled_target == b200_target
    torch.testing.assert_close(o.cpu().float(), ref_o.float(), atol=5e-3, rtol=1e-2)
    assert torch.equal(args[3].cpu(), ref_kp)
