"""Pins ``oracle/gqa_oracle.py`` against fixtures produced by the reference's own code
(``tests/golden/make_golden.py``).  CPU only."""

import json
import os

import numpy as np
import pytest
import torch

from oracle import gqa_oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
G = np.load(os.path.join(HERE, "golden", "gqa_golden.npz"))


def t(name):
    return torch.from_numpy(G[name])


def bf16(name):
    return torch.from_numpy(G[name].view(np.int16)).view(torch.bfloat16)


def fp16(name):
    return torch.from_numpy(G[name].view(np.int16)).view(torch.float16)


def test_decode_cfg1_matches_reference():
    o = O.decode_ref(t("dec_q"), t("dec_k"), t("dec_v"))
    torch.testing.assert_close(o, t("dec_o"), atol=1e-6, rtol=1e-5)


def test_decode_scale_and_softcap():
    q, k, v = t("dec_q"), t("dec_k"), t("dec_v")
    torch.testing.assert_close(O.decode_ref(q, k, v, sm_scale=0.25), t("dec_o_scale025"), atol=1e-6, rtol=1e-5)
    torch.testing.assert_close(O.decode_ref(q, k, v, softcap=2.0), t("dec_o_softcap2"), atol=1e-6, rtol=1e-5)


def test_decode_bf16_bit_identical():
    q, k, v = t("dec_q").bfloat16(), t("dec_k").bfloat16(), t("dec_v").bfloat16()
    o = O.decode_ref(q, k, v)
    # same fp32 arithmetic, same final cast: at most one bf16 ulp apart from matmul order
    torch.testing.assert_close(o.float(), bf16("dec_o_bf16").float(), atol=2e-3, rtol=8e-3)


def test_paged_decode_matches_reference():
    q, k, v = t("paged_q"), t("paged_k"), t("paged_v")
    lens, bt, page = t("paged_lens"), t("paged_bt"), int(G["paged_page"])
    o = O.paged_decode_ref(q.bfloat16(), k.bfloat16(), v.bfloat16(), lens, bt, page)
    torch.testing.assert_close(o.float(), bf16("paged_o_bf16").float(), atol=2e-3, rtol=8e-3)
    o = O.paged_decode_ref(q.half(), k.half(), v.half(), lens, bt, page)
    torch.testing.assert_close(o.float(), fp16("paged_o_fp16").float(), atol=5e-4, rtol=1e-3)
    o = O.paged_decode_ref(q, k, v, lens, bt, page, softcap=2.0)
    torch.testing.assert_close(o, t("paged_o_softcap2"), atol=1e-6, rtol=1e-5)


def test_paged_gather_bit_exact_and_ignores_unnamed_pages():
    k = G["paged_k"]
    lens, bt, page = G["paged_lens"], G["paged_bt"], int(G["paged_page"])
    for b in range(len(lens)):
        got = O.paged_gather(k, bt[b], lens[b], page)
        rows = O.physical_rows(bt[b], lens[b], page)
        assert got.shape[0] == lens[b]
        want = np.stack([k[bt[b, i // page] * page + i % page] for i in range(lens[b])])
        assert np.array_equal(got, want) and np.array_equal(k[rows], want)
    assert O.paged_gather(k, bt[0], 0, page).shape[0] == 0


def test_prefill_matches_reference():
    q, k, v = t("pre_q"), t("pre_k"), t("pre_v")
    torch.testing.assert_close(O.prefill_ref(q, k, v, True), t("pre_o_causal"), atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(O.prefill_ref(q, k, v, False), t("pre_o_full"), atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(O.prefill_ref(q, k, v, True, sm_scale=0.125, softcap=2.0),
                               t("pre_o_causal_softcap"), atol=2e-6, rtol=1e-5)
    o = O.prefill_ref(q.bfloat16(), k.bfloat16(), v.bfloat16(), True)
    torch.testing.assert_close(o.float(), bf16("pre_o_causal_bf16").float(), atol=4e-3, rtol=8e-3)
    Sq = q.shape[1]
    o, lse = O.prefill_ref(q, k[:, :Sq], v[:, :Sq], True, return_lse=True)
    torch.testing.assert_close(o, t("pre_o_square"), atol=2e-6, rtol=1e-5)
    torch.testing.assert_close(lse, t("pre_lse_square"), atol=1e-5, rtol=1e-5)


def test_prefill_packed_matches_reference_varlen():
    q, k, v = t("pre_q")[0], t("pre_k")[0], t("pre_v")[0]
    o = O.prefill_packed_ref(q, k, v, t("pre_cu_q"), t("pre_cu_k"), True)
    torch.testing.assert_close(o, t("pre_o_varlen"), atol=2e-6, rtol=1e-5)


def _paged_prefill_args():
    return (t("pp_q"), t("pp_k_new"), t("pp_v_new"), t("pp_k_pages"), t("pp_v_pages"), t("pp_cu"),
            t("pp_cache"), t("pp_bt"), int(G["pp_page"]))


def test_paged_prefill_matches_reference_and_appends():
    args = _paged_prefill_args()
    o, kp, vp = O.prefill_paged_ref(*args, is_causal=True)
    torch.testing.assert_close(o, t("pp_o_causal"), atol=2e-6, rtol=1e-5)
    assert torch.equal(kp, t("pp_k_pages_after")) and torch.equal(vp, t("pp_v_pages_after"))
    o, _, _ = O.prefill_paged_ref(*args, is_causal=False)
    torch.testing.assert_close(o, t("pp_o_full"), atol=2e-6, rtol=1e-5)
    o, _, _ = O.prefill_paged_ref(*args, is_causal=True, softcap=2.0)
    torch.testing.assert_close(o, t("pp_o_softcap"), atol=2e-6, rtol=1e-5)
    q, kn, vn, kpg, vpg = (x.half() for x in args[:5])
    o, _, _ = O.prefill_paged_ref(q, kn, vn, kpg, vpg, *args[5:], is_causal=True)
    torch.testing.assert_close(o.float(), fp16("pp_o_causal_f16").float(), atol=1e-3, rtol=1e-3)


@pytest.mark.parametrize("name,causal,wl,wr", [("c_l17", True, 17, -1), ("n_l8_r5", False, 8, 5),
                                                ("n_r11", False, -1, 11), ("c_l0", True, 0, -1)])
def test_sliding_window_matches_reference(name, causal, wl, wr):
    o = O.prefill_ref(t("sw_q"), t("sw_k"), t("sw_v"), causal, window_left=wl, window_right=wr)
    torch.testing.assert_close(o, t("sw_o_" + name), atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("name,causal,wl,wr", [("c_l9", True, 9, -1), ("n_l4_r6", False, 4, 6)])
def test_sliding_window_packed_matches_reference(name, causal, wl, wr):
    o = O.prefill_packed_ref(t("swv_q"), t("swv_k"), t("swv_v"), t("swv_cu_q"), t("swv_cu_k"), causal,
                             window_left=wl, window_right=wr)
    torch.testing.assert_close(o, t("swv_o_" + name), atol=2e-6, rtol=1e-5)


@pytest.mark.parametrize("name,rd", [("full", 32), ("partial", 16)])
def test_rope_neox_matches_reference_bit_for_bit(name, rd):
    cos, sin = O.rope_tables_ref(rd, 134, dtype=torch.float16)
    assert torch.equal(cos, fp16("rope_cos_" + name)) and torch.equal(sin, fp16("rope_sin_" + name))
    cu = torch.tensor([0, 17, 50], dtype=torch.int32)
    cache = torch.tensor([37, 100], dtype=torch.int32)
    y = O.rope_neox_packed_ref(fp16("rope_x"), cos, sin, cu, cache, rotary_dim=rd)
    assert torch.equal(y, fp16("rope_y_" + name))


def _fp8(name):
    return torch.from_numpy(G[name]).view(torch.float8_e4m3fn)


def test_paged_prefill_fp8_cache_matches_reference_expressions():
    o, kp, vp = O.prefill_paged_fp8_cache_ref(
        fp16("p8_q"), fp16("p8_k_new"), fp16("p8_v_new"), _fp8("p8_k_pages"), _fp8("p8_v_pages"), t("p8_k_scale"),
        t("p8_v_scale"), t("p8_cu"), t("p8_cache"), t("p8_bt"), int(G["p8_page"]))
    torch.testing.assert_close(o.float(), fp16("p8_o").float(), atol=1e-3, rtol=1e-3)
    assert torch.equal(kp.view(torch.uint8), _fp8("p8_k_pages_after").view(torch.uint8))
    assert torch.equal(vp.view(torch.uint8), _fp8("p8_v_pages_after").view(torch.uint8))


def test_bottom_right_known_answer():
    # tests/ops/attention/test_gqa.py:417-443 in the reference
    q = torch.zeros(1, 128, 4, 64); k = torch.zeros(1, 256, 2, 64); v = torch.zeros(1, 256, 2, 64)
    q[..., 0] = 1; k[..., 0] = 1; v[:, :128, :, 0] = 1; v[:, 128:, :, 0] = 100
    o = O.prefill_ref(q, k, v, True)
    assert o[0, 0, 0, 0] < 2 and o[0, -1, 0, 0] > 40
    assert abs(float(o[0, 0, 0, 0]) - float(G["kat_first"])) < 1e-5
    assert abs(float(o[0, -1, 0, 0]) - float(G["kat_last"])) < 1e-4


def test_fp8_quantiser_bit_exact_with_reference_function():
    x = torch.from_numpy(G["fp8_x"].view(np.int16)).view(torch.bfloat16)   # [P,page,Hkv,D]
    P, page, Hkv, D = x.shape
    xq, scale = O.quantize_kv_per_page(x.reshape(P * page, Hkv, D), page)
    assert np.array_equal(xq.view(torch.uint8).numpy().reshape(P, page, Hkv, D), G["fp8_q"])
    assert np.array_equal(scale.numpy(), G["fp8_scale"])
    dq = O.dequantize_kv_per_page(xq, scale, page, torch.bfloat16)
    assert np.array_equal(dq.view(torch.int16).numpy().view(np.uint16).reshape(P, page, Hkv, D), G["fp8_dq_bf16"])


def test_roofline_formulas_match_reference():
    R = json.load(open(os.path.join(HERE, "golden", "roofline_golden.json")))
    assert list(O.gqa_decode_roofline_ref(2, 8, 2, 256, 64, torch.float32)) == R["cfg1_decode"]
    assert list(O.gqa_fwd_roofline_ref(4, 4096, 32, 8, 128, True, torch.bfloat16)) == R["cfg2_fwd"]
    assert R["cfg2_fwd"] == [549755813888, 335544320]
    assert list(O.gqa_fwd_roofline_ref(2, 512, 64, 8, 128, False, torch.float16)) == R["fwd_noncausal_fp16"]
    assert list(O.gqa_decode_roofline_ref(32, 32, 8, 4096, 128, torch.float16)) == R["decode_llama8b_4k"]
    assert list(O.gqa_decode_paged_roofline_ref(32, 32, 8, 4096, 128, 64, torch.float16)) == R["paged_probe"]
    assert list(O.gqa_decode_paged_roofline_ref(128, 64, 8, 524288, 128, 64, torch.float8_e4m3fn)) == R["cfg4_paged_fp8"]
    assert list(O.gqa_decode_paged_roofline_ref(8, 32, 8, 1048576, 128, 128, torch.bfloat16)) == R["cfg5_paged"]


def test_merge_partials_equals_unsplit():
    torch.manual_seed(0)
    B, H, Hkv, S, D = 2, 8, 2, 96, 32
    q, k, v = torch.randn(B, H, D), torch.randn(B, S, Hkv, D), torch.randn(B, S, Hkv, D)
    full, lse_full = O.decode_ref(q, k, v, return_lse=True)
    cuts = [0, 17, 17, 64, 96]   # includes an empty shard
    os_, ls_ = [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        if a == b:
            os_.append(torch.zeros(B, H, D)); ls_.append(torch.full((B, H), float("-inf")))
        else:
            o, l = O.decode_ref(q, k[:, a:b], v[:, a:b], return_lse=True)
            os_.append(o); ls_.append(l)
    o, lse = O.merge_partials_ref(torch.stack(os_), torch.stack(ls_))
    torch.testing.assert_close(o, full, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(lse, lse_full, atol=1e-5, rtol=1e-5)
    o, lse = O.merge_partials_ref(torch.zeros(2, B, H, D), torch.full((2, B, H), -1e30))
    assert torch.all(o == 0)
