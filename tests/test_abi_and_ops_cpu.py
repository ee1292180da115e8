"""CPU-only tests: the C-ABI library loads and exports every declared symbol; the op layer
(validation, kernel selection, kernel_map overrides, plugin targets, roofline) behaves like the
reference's, exercised with stand-in kernels that launch nothing."""

import ctypes
import json
import os
import re
import subprocess
import sys

import pytest
import torch

import tileops_b200
from tileops_b200 import _native, backend
from tileops_b200.backend import registry
from tileops_b200.kernels import Kernel, gqa_decode_paged_block_ns
from tileops_b200.kernels.call_spec import AttentionCall
from tileops_b200.ops import (
    GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp,
    GroupedQueryAttentionDecodePagedWithKVCacheFwdOp,
    GroupedQueryAttentionDecodeWithKVCacheFwdOp,
    GroupedQueryAttentionFwdOp,
    GroupedQueryAttentionPrefillFwdOp,
)
from tileops_b200.ops.selection import PAGED_DECODE_KEYS
from tileops_b200.perf import formulas, load_profile

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---------------------------------------------------------------------------- C ABI
def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "tileops_b200.h")).read()
    declared = set(re.findall(r"\b(tb200_[a-z0-9_]+)\s*\(", header))
    declared -= {"tb200_status", "tb200_dtype"}
    assert declared == set(_native.SIGNATURES), (declared, set(_native.SIGNATURES))
    lib = _native.lib()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.tb200_version() >= 1


def test_abi_rejects_bad_arguments_without_touching_a_gpu():
    lib = _native.lib()
    assert lib.tb200_gqa_decode_workspace_bytes(0, 32, 8, 128) == 0
    assert lib.tb200_gqa_decode_workspace_bytes(4, 30, 8, 128) == 0
    assert lib.tb200_gqa_decode_workspace_bytes(64, 32, 8, 128) > 0
    st = lib.tb200_gqa_decode(None, None, None, None, None, None, 0, None, 0, None, None, 1, 1, 1,
                              1, 8, 2, 64, 16, 128, 64, 0, 1.0, 0.0, 0, 0, None, 0, None)
    assert st == 1 and b"non-null" in lib.tb200_last_error()
    buf = ctypes.create_string_buffer(64)
    p = ctypes.addressof(buf)
    st = lib.tb200_gqa_decode(p, p, p, p, None, None, 16, None, 0, None, None, 1, 1, 1,
                              1, 8, 3, 64, 16, 128, 64, 0, 1.0, 0.0, 0, 0, None, 0, None)
    assert st == 1 and b"divisible" in lib.tb200_last_error()
    st = lib.tb200_gqa_decode(p, p, p, p, None, None, 16, None, 0, None, None, 1, 1, 1,
                              1, 8, 2, 96, 16, 192, 96, 0, 1.0, 0.0, 0, 0, None, 0, None)
    assert st == 2 and b"head dim" in lib.tb200_last_error()
    st = lib.tb200_gqa_lse_merge(None, None, None, None, 2, 4, 64, 0, 0, 3, None)
    assert st == 1


# ---------------------------------------------------------------------------- op layer
class _Recorder(Kernel):
    """Stand-in kernel: answers selection, compiles and launches nothing."""
    supported_archs = None
    general = True
    built = []

    def __init__(self, *args, **kwargs):
        self.args, self.kwargs = args, kwargs
        self.config = {}
        type(self).built.append(self)

    def forward(self, q, *rest, **kw):
        self.last = (q, rest)
        return torch.zeros_like(q)


def test_constructor_validation_messages():
    with pytest.raises(ValueError, match="heads must be divisible by heads_kv"):
        GroupedQueryAttentionDecodeWithKVCacheFwdOp(1, 30, 8, 128, 64)
    with pytest.raises(ValueError, match="heads_kv must be positive"):
        GroupedQueryAttentionDecodeWithKVCacheFwdOp(1, 8, 0, 128, 64)
    with pytest.raises(ValueError, match="softcap must be non-negative"):
        GroupedQueryAttentionDecodeWithKVCacheFwdOp(1, 8, 2, 128, 64, softcap=-1.0)
    with pytest.raises(ValueError, match="page_size must be positive"):
        GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(1, 8, 2, 128, 64, 0)
    with pytest.raises(ValueError, match="seq_len must be positive"):
        GroupedQueryAttentionFwdOp(1, 8, 2, 0, 64)
    with pytest.raises(ValueError, match="causal prefill requires max_seqlen_q <= max_seqlen_kv"):
        GroupedQueryAttentionPrefillFwdOp(1, 8, 2, 64, 128, 64)
    with pytest.raises(ValueError, match="backend must be one of"):
        GroupedQueryAttentionPrefillFwdOp(1, 8, 2, 64, 64, 64, backend="nope")
    with pytest.raises(ValueError, match="requires validate_uniform_cu_seqlens=True"):
        GroupedQueryAttentionPrefillFwdOp(1, 8, 2, 64, 64, 64, validate_uniform_cu_seqlens=False)
    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(2, 8, 2, 256, 64)
    assert op.sm_scale == 64 ** -0.5 and op.softcap == 0.0


def test_construction_needs_no_device_and_selection_reports_arch():
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(1, 16, 4, 1024, 128, 64)
    assert set(op.kernel_map) == {"gqa_decode_paged_kernel"}
    if not torch.cuda.is_available():
        with pytest.raises(ValueError, match="no implementation serves this call"):
            op._get_kernel((), torch.float16)
    with pytest.raises(ValueError, match="Expected dtype torch.float16 or torch.bfloat16"):
        op._get_kernel((), torch.float32)


@pytest.mark.parametrize("page_size", [96, 160, 224])
def test_paged_rejects_unsupported_page_tile(page_size):
    # tests/ops/attention/test_gqa_decode_paged.py:143-151 in the reference
    with pytest.raises(ValueError, match="matches no supported block_N"):
        gqa_decode_paged_block_ns(page_size)
    assert gqa_decode_paged_block_ns(192) == (64,)
    assert gqa_decode_paged_block_ns(16) == (16,)
    assert gqa_decode_paged_block_ns(256) == (64,)


def test_kernel_map_override_is_what_gets_built_positionally():
    _Recorder.built.clear()
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(
        2, 8, 2, 256, 64, 16, sm_scale=0.25, softcap=2.0, kernel_map={"gqa_decode_paged_kernel": _Recorder})
    assert op._overridden_keys == {"gqa_decode_paged_kernel"}
    q = torch.zeros(2, 8, 64, dtype=torch.bfloat16)
    k = torch.zeros(256, 2, 64, dtype=torch.bfloat16)
    lens = torch.zeros(2, dtype=torch.int32)
    bt = torch.zeros(2, 16, dtype=torch.int32)
    out = op(q, k, k, lens, bt)
    assert out.shape == q.shape
    (kern,) = _Recorder.built
    assert kern.args == (2, 8, 2, 256, 64, 16, torch.bfloat16)
    assert kern.kwargs == {"sm_scale": 0.25, "softcap": 2.0, "tune": False}
    op(q, k, k, lens, bt)
    assert len(_Recorder.built) == 1                       # cached per dtype
    op(q.half(), k.half(), k.half(), lens, bt)
    assert len(_Recorder.built) == 2
    assert op.eval_roofline() == formulas.gqa_decode_paged_roofline(
        batch=2, heads=8, heads_kv=2, seqlen_kv=256, dim=64, page_size=16, dtype=torch.float16)


def test_refused_override_is_an_error_never_replaced():
    class Refuses(_Recorder):
        supported_archs = [1]

    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(1, 8, 2, 64, 64, kernel_map={"gqa_decode_kernel": Refuses})
    with pytest.raises(ValueError, match="the kernel supplied for gqa_decode_kernel"):
        op._get_kernel((), torch.float16)


def test_ambiguous_dispatch_is_reported():
    class Special(_Recorder):
        general = False

    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(1, 8, 2, 64, 64, 16)
    op.kernel_map = {"gqa_decode_paged_bs1_kernel": Special, "gqa_decode_paged_kernel": Special}
    with pytest.raises(ValueError, match="dispatch is ambiguous"):
        op.select_kernel_key(PAGED_DECODE_KEYS, AttentionCall(arch=100, dtype=torch.float16))
    op.kernel_map = {"gqa_decode_paged_bs1_kernel": Special, "gqa_decode_paged_kernel": _Recorder}
    assert op.select_kernel_key(PAGED_DECODE_KEYS, AttentionCall(arch=100)) == "gqa_decode_paged_bs1_kernel"


def test_decode_op_validates_dtypes_and_passes_live_length():
    _Recorder.built.clear()
    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(2, 8, 2, 256, 64, kernel_map={"gqa_decode_kernel": _Recorder})
    q = torch.zeros(2, 8, 64, dtype=torch.float16)
    k = torch.zeros(2, 100, 2, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="input 'k' has dtype torch.bfloat16, expected 'same_as\\(q\\)'"):
        op(q, k.bfloat16(), k)
    with pytest.raises(ValueError, match="input 'q' has dtype torch.float32"):
        op(q.float(), k.float(), k.float())
    op(q, k, k)
    assert _Recorder.built[-1].last[1][2] == 100           # real_seqlen_kv, no padding copy
    assert _Recorder.built[-1].args == (2, 8, 2, 256, 64, torch.float16)


def test_fwd_op_shape_errors_and_packed_views():
    _Recorder.built.clear()
    op = GroupedQueryAttentionFwdOp(2, 8, 2, 16, 64, kernel_map={"gqa_prefill_fwd_kernel": _Recorder})
    q = torch.zeros(2, 16, 8, 64, dtype=torch.bfloat16)
    k = torch.zeros(2, 16, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match=r"q must have shape \(2, 16, 8, 64\)"):
        op(q[:, :8], k, k)
    with pytest.raises(ValueError, match=r"v must have shape"):
        op(q, k, k[:1])
    out = op(q, k, k)
    assert out.shape == q.shape
    kern = _Recorder.built[-1]
    assert kern.kwargs["max_seqlen_q"] == 16 and kern.kwargs["is_causal"] is True
    assert kern.kwargs["accum_dtype"] == torch.float32 and kern.kwargs["dtype"] == torch.bfloat16
    packed_q, rest = kern.last
    assert packed_q.shape == (32, 8, 64) and rest[0].shape == (32, 2, 64)
    assert rest[2].tolist() == [0, 16, 32] and rest[2].dtype == torch.int32
    assert op.eval_roofline() == formulas.gqa_fwd_roofline(
        batch=2, seq_len=16, heads=8, heads_kv=2, dim=64, is_causal=True, dtype=torch.bfloat16)


def test_fp8_paged_op_contract():
    _Recorder.built.clear()
    op = GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp(
        1, 8, 2, 64, 64, 16, kernel_map={"gqa_decode_paged_fp8_kernel": _Recorder})
    q = torch.zeros(1, 8, 64, dtype=torch.bfloat16)
    kf = torch.zeros(64, 2, 64, dtype=torch.float8_e4m3fn)
    sc = torch.ones(4, 2)
    lens = torch.zeros(1, dtype=torch.int32)
    bt = torch.zeros(1, 4, dtype=torch.int32)
    with pytest.raises(ValueError, match="input 'k' has dtype torch.bfloat16"):
        op(q, kf.to(torch.bfloat16), kf, sc, sc, lens, bt)
    with pytest.raises(ValueError, match=r"k_scale must have shape \(4, 2\)"):
        op(q, kf, kf, sc[:2], sc, lens, bt)
    op(q, kf, kf, sc, sc, lens, bt)
    flops, nbytes = op.eval_roofline()
    assert nbytes == formulas.gqa_decode_paged_roofline(
        batch=1, heads=8, heads_kv=2, seqlen_kv=64, dim=64, page_size=16, dtype=torch.float8_e4m3fn)[1]


# ---------------------------------------------------------------------------- plugin seam
@pytest.fixture
def clean_registry():
    state = registry.snapshot()
    yield
    registry.restore(state)


def test_backend_target_builder_receives_specs_and_params(clean_registry):
    calls = []

    def build(q, k, v, real_seqlen_kv, block_table, *, page_size, sm_scale, softcap):
        calls.append((q, k, block_table, page_size, sm_scale, softcap))
        return lambda *tensors: torch.full_like(tensors[0], 7)

    backend.register_detector("fake", lambda device: device.type == "cpu")
    backend.register_kernel_builder("GroupedQueryAttentionDecodePagedWithKVCacheFwdOp", "fake", build)
    with pytest.raises(backend.BackendError):
        backend.register_kernel_builder("GroupedQueryAttentionDecodePagedWithKVCacheFwdOp", "fake", build)
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(1, 8, 2, 64, 64, 16, softcap=3.0)
    q = torch.zeros(1, 8, 64, dtype=torch.float16)
    k = torch.zeros(64, 2, 64, dtype=torch.float16)
    out = op(q, k, k, torch.zeros(1, dtype=torch.int32), torch.zeros(1, 4, dtype=torch.int32))
    assert float(out[0, 0, 0]) == 7 and op._settled_target == "fake"
    spec_q, spec_k, spec_bt, page, scale, cap = calls[0]
    assert spec_q == backend.TensorSpec(torch.device("cpu"), torch.float16, (1, 8, 64))
    assert spec_bt.dtype == torch.int32 and page == 16 and cap == 3.0 and scale == 64 ** -0.5
    op(q, k, k, torch.zeros(1, dtype=torch.int32), torch.zeros(1, 4, dtype=torch.int32))
    assert len(calls) == 1                                  # memoised per (device, dtypes, shapes)
    with pytest.raises(backend.UnknownTargetError):
        backend.set_default_target("nobody")
    op2 = GroupedQueryAttentionDecodeWithKVCacheFwdOp(1, 8, 2, 64, 64)
    with pytest.raises(backend.OpNotAvailableError):
        op2(q, torch.zeros(1, 64, 2, 64, dtype=torch.float16), torch.zeros(1, 64, 2, 64, dtype=torch.float16))
    assert op2._settled_target is None                      # a failed first call settles nothing


def test_b200_plugin_registers_a_detector_and_a_builder_per_op(clean_registry):
    from tileops_b200 import plugin
    plugin.register(backend)
    assert plugin.TARGET in registry.known_targets()
    assert registry.DETECTORS[plugin.TARGET] is plugin.detect
    assert plugin.detect(torch.device("cpu")) is False
    m = tileops_b200.manifest.load_manifest()
    for op_name, builder in plugin.BUILDERS.items():
        assert op_name in m and registry.BUILDERS[(op_name, plugin.TARGET)] is builder
    with pytest.raises(backend.BackendError):
        plugin.register(backend)                            # one detector per target
    # builders are described with specs and manifest params only; nothing touches a device
    spec = backend.TensorSpec
    q = spec(torch.device("cuda", 0), torch.bfloat16, (4, 32, 128))
    kv = spec(torch.device("cuda", 0), torch.bfloat16, (4096, 8, 128))
    meta = spec(torch.device("cuda", 0), torch.int32, (4,))
    assert callable(plugin.build_paged_decode(q, kv, kv, meta, meta, page_size=64, sm_scale=None, softcap=None))
    with pytest.raises(ValueError, match="cache of q's element type"):
        plugin.build_paged_prefill(q, q, q, spec(kv.device, torch.float8_e4m3fn, kv.shape), kv, page_size=64)
    text = open(os.path.join(ROOT, "pyproject.toml")).read()
    assert '[project.entry-points."tileops.backends"]' in text and 'b200 = "tileops_b200.plugin"' in text


def test_mha_decode_rows_map_onto_a_gqa_group():
    from tileops_b200.kernels.mha_decode import _as_groups, _from_groups
    from tileops_b200.ops import MultiHeadAttentionDecodePagedWithKVCacheFwdOp, MultiHeadAttentionDecodeWithKVCacheFwdOp
    from oracle import gqa_oracle as O
    g = torch.Generator().manual_seed(3)
    B, Sq, H, D, S = 2, 3, 4, 16, 40
    q = torch.randn(B, Sq, H, D, generator=g)
    k = torch.randn(B, S, H, D, generator=g)
    v = torch.randn(B, S, H, D, generator=g)
    # the q rows of one head, laid out as the q-head group of that KV head, give plain per-head attention
    o = _from_groups(O.decode_ref(_as_groups(q), k, v), B, Sq, H, D)
    want = torch.softmax(torch.einsum("bqhd,bkhd->bhqk", q, k) * D ** -0.5, dim=-1)
    want = torch.einsum("bhqk,bkhd->bqhd", want, v)
    torch.testing.assert_close(o, want, atol=1e-5, rtol=1e-5)
    assert _as_groups(q[:, :1]).shape == (B, H, D)
    op = MultiHeadAttentionDecodeWithKVCacheFwdOp(B, H, Sq, 64, D)
    assert list(op.kernel_map) == ["mha_decode_kernel"]
    with pytest.raises(ValueError, match="more than seqlen_kv"):
        op(q, torch.zeros(B, 65, H, D), torch.zeros(B, 65, H, D))
    assert list(MultiHeadAttentionDecodePagedWithKVCacheFwdOp(B, H, 1, 128, 64, 64).kernel_map) == [
        "mha_decode_paged_kernel"]


def test_manifest_and_profile():
    m = tileops_b200.manifest.load_manifest()
    for name in ("GroupedQueryAttentionFwdOp", "GroupedQueryAttentionPrefillFwdOp",
                 "GroupedQueryAttentionDecodeWithKVCacheFwdOp",
                 "GroupedQueryAttentionDecodePagedWithKVCacheFwdOp"):
        assert m[name]["status"] == "implemented" and m[name]["roofline"]["func"].startswith("tileops.perf.formulas.")
    assert list(m["GroupedQueryAttentionDecodePagedWithKVCacheFwdOp"]["signature"]["inputs"]) == [
        "q", "k", "v", "real_seqlen_kv", "block_table"]
    assert GroupedQueryAttentionDecodePagedWithKVCacheFwdOp.__manifest_param_names__ == (
        "page_size", "sm_scale", "softcap")
    prof = load_profile("b200")
    assert prof["arch"] == 100 and float(prof["hbm"]["effective"]) > 6e12


def test_product_formulas_match_reference_values():
    R = json.load(open(os.path.join(ROOT, "tests", "golden", "roofline_golden.json")))
    F = formulas
    assert list(F.gqa_decode_roofline(q_shape=(2, 8, 64), kv_shape=(2, 256, 2, 64), dtype=torch.float32)) == R["cfg1_decode"]
    assert list(F.gqa_fwd_roofline(q_shape=(4, 4096, 32, 128), kv_shape=(4, 4096, 8, 128), is_causal=True,
                                   dtype=torch.bfloat16)) == R["cfg2_fwd"]
    assert list(F.gqa_fwd_roofline(batch=2, seq_len=512, heads=64, heads_kv=8, dim=128, is_causal=False,
                                   dtype=torch.float16)) == R["fwd_noncausal_fp16"]
    assert list(F.gqa_decode_roofline(q_shape=(32, 32, 128), kv_shape=(32, 4096, 8, 128), dtype=torch.float16)) == R["decode_llama8b_4k"]
    assert list(F.gqa_decode_paged_roofline(q_shape=(32, 32, 128), kv_shape=(4096, 8, 128), page_size=64,
                                            dtype=torch.float16)) == R["paged_probe"]
    assert list(F.gqa_decode_paged_roofline(q_shape=(128, 64, 128), kv_shape=(524288, 8, 128), page_size=64,
                                            dtype=torch.float8_e4m3fn)) == R["cfg4_paged_fp8"]
    assert list(F.gqa_decode_paged_roofline(q_shape=(8, 32, 128), kv_shape=(1048576, 8, 128), page_size=128,
                                            dtype=torch.bfloat16)) == R["cfg5_paged"]
    assert list(F.gqa_prefill_varlen_fwd_roofline(
        q_shape=(1024, 32, 128), k_shape=(8192, 8, 128), batch=2, max_seqlen_q=512, max_seqlen_kv=4096,
        q_lens=[512, 512], kv_lens=[4096, 4096], is_causal=True, dtype=torch.bfloat16)) == R["varlen_packed"]
    assert list(F.gqa_prefill_varlen_fwd_roofline(
        q_shape=(40, 4, 32), k_shape=(72, 2, 32), batch=2, max_seqlen_q=24, max_seqlen_kv=50,
        q_lens=[24, 16], kv_lens=[50, 22], is_causal=True, dtype=torch.float16)) == R["varlen_ragged"]


def test_paged_prefill_formula_matches_reference_values_and_manifest_workloads():
    R = json.load(open(os.path.join(ROOT, "tests", "golden", "roofline_golden.json")))
    F = formulas.gqa_prefill_paged_with_kv_cache_fwd_roofline
    assert list(F(total_q=4096, batch=8, q_lens=[512] * 8, cache_lens=[4096] * 8, heads=32, heads_kv=8, dim=128,
                  page_size=64, max_pages_per_req=72, max_seqlen_q=512, is_causal=True,
                  dtype=torch.float16)) == R["paged_prefill_llama8b"]
    assert list(F(total_q=4608, batch=8, q_lens=[256, 512, 768, 1024, 384, 640, 896, 128],
                  cache_lens=[4096, 8192, 16384, 32768, 12288, 24576, 30720, 2048], heads=32, heads_kv=8,
                  dim=128, page_size=64, max_pages_per_req=528, max_seqlen_q=1024, is_causal=True,
                  dtype=torch.bfloat16)) == R["paged_prefill_mixed"]
    assert list(F(total_q=2048, batch=4, heads=8, heads_kv=2, dim=64, page_size=64, max_pages_per_req=72,
                  max_seqlen_q=512, is_causal=False, dtype=torch.float16)) == R["paged_prefill_aggregate_only"]
    entry = tileops_b200.manifest.load_manifest()["GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp"]
    assert entry["roofline"]["func"].endswith("gqa_prefill_paged_with_kv_cache_fwd_roofline")
    for w in entry["workloads"]:
        flops, nbytes = F(**w)
        assert flops > 0 and nbytes > 0 and sum(w["q_lens"]) == w["total_q"]


def test_paged_prefill_op_constructor_and_selection_follow_the_reference():
    from tileops_b200.ops import (GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp as PagedOp,
                                  GroupedQueryAttentionPrefillVarlenFwdOp as VarlenOp)
    with pytest.raises(ValueError, match="page_size must be a power of two"):
        PagedOp(2, 8, 2, 8, 48, 64)
    with pytest.raises(ValueError, match="max_position is required when fuse_rope=True"):
        PagedOp(2, 8, 2, 8, 64, 64, fuse_rope=True)
    with pytest.raises(ValueError, match="rotary_dim requires fuse_rope=True"):
        PagedOp(2, 8, 2, 8, 64, 64, rotary_dim=32)
    with pytest.raises(ValueError, match="max_pages_per_req must be positive"):
        PagedOp(2, 8, 2, 0, 64, 64)
    op = PagedOp(2, 8, 2, 8, 64, 64, softcap=50.0)
    assert op.max_cache_len == 512 and op.groups == 4 and op.softcap == 50.0
    assert sorted(op.kernel_map) == ["gqa_prefill_paged_with_fp8_kv_cache_fwd_kernel",
                                     "gqa_prefill_paged_with_kv_cache_fwd_kernel",
                                     "gqa_prefill_paged_with_kv_cache_rope_fwd_kernel"]
    from tileops_b200.ops.selection import PAGED_PREFILL_KEYS
    import dataclasses

    def on_sm100(call):   # no GPU in the CPU suite: state the architecture in the call
        return dataclasses.replace(call, arch=100)
    assert op.select_kernel_key(PAGED_PREFILL_KEYS, on_sm100(op.attention_call(torch.float16))) == \
        "gqa_prefill_paged_with_kv_cache_fwd_kernel"
    # pages below 16 tokens and head dims other than 64 / 128 / 256 have no sm_100 implementation
    rope = PagedOp(2, 8, 2, 8, 64, 64, fuse_rope=True, max_position=512, rotary_dim=32)
    assert rope.select_kernel_key(PAGED_PREFILL_KEYS, on_sm100(rope.attention_call(torch.float16))) == \
        "gqa_prefill_paged_with_kv_cache_rope_fwd_kernel"
    cos, sin = rope._get_rope_cos_sin(torch.device("cpu"), torch.float16)
    assert cos.shape == (512, 16) and cos.dtype == torch.float16 and float(cos[0, 0]) == 1.0 and float(sin[0, 0]) == 0.0
    f8op = PagedOp(2, 8, 2, 8, 64, 64, cache_dtype=torch.float8_e4m3fn)
    assert f8op.select_kernel_key(PAGED_PREFILL_KEYS, on_sm100(f8op.attention_call(torch.float16))) == \
        "gqa_prefill_paged_with_fp8_kv_cache_fwd_kernel"
    for bad in (PagedOp(2, 8, 2, 64, 8, 64), PagedOp(2, 8, 2, 8, 64, 96)):
        with pytest.raises(ValueError, match="no implementation serves this call"):
            bad.select_kernel_key(PAGED_PREFILL_KEYS, on_sm100(bad.attention_call(torch.float16)))
    with pytest.raises(NotImplementedError):
        op.total_flops
    q = torch.zeros(4, 8, 64, dtype=torch.float16)
    with pytest.raises(ValueError, match="q must be on a cuda device"):
        op(q, q, q, q, q, q, q, q, q, q, 4)
    v = VarlenOp(2, 8, 2, 64, 128, 256)
    assert list(v.kernel_map) == ["gqa_prefill_varlen_fwd_kernel"]
    with pytest.raises(ValueError, match="q must be a CUDA tensor"):
        v(q, q, q, q, q)
    with pytest.raises(RuntimeError, match="requires a prior forward"):
        v.eval_roofline()


def test_packed_prefill_op_routes_ragged_requests_to_the_varlen_kernel():
    from tileops_b200.ops import GroupedQueryAttentionPrefillFwdOp
    from tileops_b200.ops.selection import PACKED_PREFILL_KEYS
    import dataclasses

    def call(op, uniform):
        return dataclasses.replace(op.attention_call(is_fp8=False, is_uniform=uniform), arch=100)
    op = GroupedQueryAttentionPrefillFwdOp(2, 8, 2, 128, 256, 256, dtype=torch.bfloat16)
    assert op.select_kernel_key(PACKED_PREFILL_KEYS, call(op, True)) == "gqa_prefill_fwd_kernel"
    assert op.select_kernel_key(PACKED_PREFILL_KEYS, call(op, False)) == "gqa_prefill_varlen_fwd_kernel"
    op = GroupedQueryAttentionPrefillFwdOp(2, 8, 2, 128, 256, 256, dtype=torch.bfloat16, backend="varlen")
    assert op.select_kernel_key(PACKED_PREFILL_KEYS, call(op, True)) == "gqa_prefill_varlen_fwd_kernel"


def test_workload_generator_shards_reproduce_the_full_problem():
    from tileops_b200 import workloads as W
    full = W.make_paged_decode(9, 2, 4, 2, 16, 8, lens=[50, 21], dtype=torch.float32, device="cpu")
    from oracle import gqa_oracle as O
    for b in range(2):
        rows = O.physical_rows(full.block_table[b].numpy(), full.lens[b], 8)
        logical = full.k[torch.from_numpy(rows)]
        parts = []
        for (p0, p1) in ((0, 3), (3, 7)):
            sh = W.make_paged_decode(9, 2, 4, 2, 16, 8, lens=[50, 21], dtype=torch.float32, device="cpu",
                                     page_begin=p0, page_end=p1)
            r = O.physical_rows(sh.block_table[b].numpy(), sh.lens[b], 8)
            parts.append(sh.k[torch.from_numpy(r)])
            assert torch.equal(sh.q, full.q)
        assert torch.equal(torch.cat(parts), logical)


# a TileOPs source tree: named by TILEOPS_SOURCE_TREE, else a checkout called "reference" beside this repository
REFERENCE_SRC = os.environ.get("TILEOPS_SOURCE_TREE", os.path.join(os.path.dirname(ROOT), "reference", "src"))


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE_SRC, "tileops", "backend")),
                    reason="needs a TileOPs source tree (present in the build container only)")
def test_plugin_registers_with_the_real_tileops_backend():
    """The plugin seam against the reference's own ``tileops.backend`` (``src/tileops/backend/registry.py:42-84``,
    ``protocol.py:10-32``), in a child process so that the reference tree never enters this process: importing
    the plugin registers the detector and the five builders in the REAL registry, this package's backend module
    is then that registry, builders answer ``(*TensorSpec, **params)``, and the real dispatch resolves the target."""
    code = r'''
import torch, tileops.backend as tb
from tileops.backend import registry, dispatch
import tileops_b200.backend as mine
assert mine.USES_INSTALLED_TILEOPS and mine.registry is registry and mine.TensorSpec is tb.TensorSpec
from tileops_b200 import plugin                      # the entry-point import: registers on import
assert registry.DETECTORS[plugin.TARGET] is plugin.detect
assert len(plugin.BUILDERS) == 5
for op_name, builder in plugin.BUILDERS.items():
    assert registry.BUILDERS[(op_name, plugin.TARGET)] is builder, op_name
assert plugin.TARGET in tb.registered_targets()
try:
    plugin.register(tb)
    raise SystemExit("a second detector for the same target must be refused")
except tb.BackendError:
    pass
S = tb.TensorSpec
dev = torch.device("cuda", 0)
q, kv, meta = S(dev, torch.bfloat16, (4, 32, 128)), S(dev, torch.bfloat16, (4096, 8, 128)), S(dev, torch.int32, (4,))
run = registry.BUILDERS[("GroupedQueryAttentionDecodePagedWithKVCacheFwdOp", plugin.TARGET)](
    q, kv, kv, meta, meta, page_size=64, sm_scale=None, softcap=None)
assert callable(run)
tb.set_default_target(plugin.TARGET)
assert tb.default_target() == plugin.TARGET
# this package's operators dispatch through the same (real) tables
from tileops_b200.ops import GroupedQueryAttentionDecodePagedWithKVCacheFwdOp
op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(4, 32, 8, 4096, 128, 64)
print("REAL-BACKEND-OK")
'''
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([REFERENCE_SRC, ROOT]))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd="/tmp", timeout=300)
    assert out.returncode == 0 and "REAL-BACKEND-OK" in out.stdout, out.stdout[-2000:] + out.stderr[-3000:]


def test_paged_decode_op_can_range_check_its_block_table(clean_registry):
    """Opt-in host-side check of lengths and page ids (the kernel trusts them): a bad table is a ValueError
    before anything is launched."""
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(2, 8, 2, 256, 64, 64, kernel_map={"gqa_decode_paged_kernel": _Recorder})
    op.validate_inputs = True
    q = torch.zeros(2, 8, 64, dtype=torch.float16)
    k = torch.zeros(256, 2, 64, dtype=torch.float16)
    lens = torch.tensor([100, 64], dtype=torch.int32)
    good = torch.tensor([[0, 1], [3, 9]], dtype=torch.int32)      # entry [1, 1] is behind sequence 1's length: not read
    op(q, k, k, lens, good)
    with pytest.raises(ValueError, match=r"block_table\[0, 1\]=7 is outside the pool of 4 pages"):
        op(q, k, k, lens, torch.tensor([[0, 7], [3, 0]], dtype=torch.int32))
    with pytest.raises(ValueError, match="needs 3 pages"):
        op(q, k, k, torch.tensor([129, 1], dtype=torch.int32), good)
    with pytest.raises(ValueError, match="non-negative"):
        op(q, k, k, torch.tensor([-1, 1], dtype=torch.int32), good)
