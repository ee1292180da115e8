"""Generate the golden fixtures in this directory from the REFERENCE's own code.

Run once in a container that has the tile-ai/TileOPs tree mounted (its path is the
first argument); the resulting ``*.npz`` / ``*.json``
files are committed and are what the CPU test-suite pins ``oracle/gqa_oracle.py``
against on machines where the reference is absent.

What is executed from the reference (imported, never copied):
  * ``workloads.attention.gqa.GroupedQueryAttentionDecodeWorkload.ref_program``
  * ``workloads.attention.gqa._compute_gqa_square_lse``
  * ``workloads.gqa_fp8_utils.quantize_kv_fa3_descale``
  * ``tests.ops.attention.test_gqa_decode_paged.GroupedQueryAttentionDecodePagedTest.ref_program``
  * ``tests.ops.attention.test_gqa._gqa_prefill_ref`` / ``_gqa_prefill_varlen_ref``
  * ``tests.ops.attention.test_gqa_prefill_paged._gqa_prefill_paged_ref`` /
    ``_fill_paged_cache_from_logical`` / ``_physical_pos``
  * ``tests.ops.attention.test_gqa_sliding_window(.py|_varlen.py)`` reference programs
  * ``tests.ops.test_rope.ref_rope_neox_position_ids`` / ``_compute_freqs_cis_base``
  * ``tileops.perf.formulas.gqa_*_roofline``
``tileops.ops`` itself needs a newer TileLang than the container has, so a stub
module carrying the handful of names those files import is placed in
``sys.modules`` first; none of the executed functions touches the stubbed names.

bf16 tensors are stored as their uint16 bit patterns, e4m3 tensors as uint8.
"""

from __future__ import annotations

import json
import os
import sys
import types

import numpy as np
import torch

if len(sys.argv) < 2:
    sys.exit("usage: make_golden.py <path to a checkout of tile-ai/TileOPs>")
REF = sys.argv[1]
HERE = os.path.dirname(os.path.abspath(__file__))
SEED = 1235  # the reference's own test seed (tests/conftest.py:45)


class _Anything(types.ModuleType):
    """Module whose every attribute is a dummy class (for names imported but unused)."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        cls = type(name, (), {"default_kernel_map": property(lambda self: {})})
        setattr(self, name, cls)
        return cls


def _install_stubs():
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(REF, "src"))
    import tileops  # noqa: F401  (package import is fine; tileops.ops is not)
    for name in ("tileops.ops", "tileops.ops.attention", "tileops.ops.attention.selection",
                 "tileops.ops.op_base", "tileops.utils", "tileops.kernels",
                 "tileops.kernels.attention"):
        if name not in sys.modules or name == "tileops.ops":
            sys.modules[name] = _Anything(name)
    sys.modules["tileops.ops.attention.selection"].DENSE_PREFILL_KEYS = ()
    sys.modules["tileops.ops.attention.selection"].PACKED_PREFILL_KEYS = ()
    sys.modules["tileops.utils"].is_h200 = lambda *a, **k: False


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float16:
        return t.view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.view(torch.uint8).numpy()
    return t.numpy()


def main():
    _install_stubs()
    from workloads.attention import gqa as wl
    from workloads import gqa_fp8_utils as fp8u

    g = torch.Generator().manual_seed(SEED)
    out = {}

    # ---- contiguous decode, the reference's CPU-runnable case (fp32 on CPU) + variants
    B, H, Hkv, S, D = 2, 8, 2, 256, 64
    q = torch.randn(B, H, D, generator=g)
    k = torch.randn(B, S, Hkv, D, generator=g)
    v = torch.randn(B, S, Hkv, D, generator=g)
    w = wl.GroupedQueryAttentionDecodeWorkload(B, H, Hkv, S, D, torch.float32)
    out["dec_q"], out["dec_k"], out["dec_v"] = q.numpy(), k.numpy(), v.numpy()
    out["dec_o"] = w.ref_program(q, k, v).numpy()
    w2 = wl.GroupedQueryAttentionDecodeWorkload(B, H, Hkv, S, D, torch.float32, sm_scale=0.25)
    out["dec_o_scale025"] = w2.ref_program(q, k, v).numpy()
    w3 = wl.GroupedQueryAttentionDecodeWorkload(B, H, Hkv, S, D, torch.float32, softcap=2.0)
    out["dec_o_softcap2"] = w3.ref_program(q, k, v).numpy()
    w4 = wl.GroupedQueryAttentionDecodeWorkload(B, H, Hkv, S, D, torch.bfloat16)
    out["dec_o_bf16"] = bits(w4.ref_program(q.bfloat16(), k.bfloat16(), v.bfloat16()))

    # ---- paged decode: permuted block table, ragged lengths, bf16 and fp16
    from tests.ops.attention import test_gqa_decode_paged as tp
    B, H, Hkv, D, page = 3, 8, 2, 64, 16
    lens = torch.tensor([37, 64, 5], dtype=torch.int32)
    pages = [-(-int(x) // page) for x in lens]
    P = sum(pages) + 2                       # two spare pages that no table names
    perm = torch.randperm(P, generator=g).to(torch.int32)
    W = max(pages) + 1
    bt = torch.zeros(B, W, dtype=torch.int32)
    off = 0
    for b in range(B):
        bt[b, :pages[b]] = perm[off:off + pages[b]]
        off += pages[b]
    qp = torch.randn(B, H, D, generator=g)
    kp = torch.randn(P * page, Hkv, D, generator=g)
    vp = torch.randn(P * page, Hkv, D, generator=g)
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float16, "fp16")):
        t = tp.GroupedQueryAttentionDecodePagedTest(B, H, Hkv, P * page, D, page, dt)
        o = t.ref_program(qp.to(dt), kp.to(dt), vp.to(dt), lens, bt)
        out[f"paged_o_{tag}"] = bits(o)
    t = tp.GroupedQueryAttentionDecodePagedTest(B, H, Hkv, P * page, D, page, torch.float32,
                                                softcap=2.0)
    out["paged_o_softcap2"] = t.ref_program(qp, kp, vp, lens, bt).numpy()
    out["paged_q"], out["paged_k"], out["paged_v"] = qp.numpy(), kp.numpy(), vp.numpy()
    out["paged_lens"], out["paged_bt"] = lens.numpy(), bt.numpy()
    out["paged_page"] = np.int32(page)

    # ---- prefill: square causal, Sq<Skv causal (bottom-right), non-causal, softcap; LSE
    from tests.ops.attention import test_gqa as tg
    B, Sq, Skv, H, Hkv, D = 2, 40, 72, 4, 2, 32
    qf = torch.randn(B, Sq, H, D, generator=g)
    kf = torch.randn(B, Skv, Hkv, D, generator=g)
    vf = torch.randn(B, Skv, Hkv, D, generator=g)
    out["pre_q"], out["pre_k"], out["pre_v"] = qf.numpy(), kf.numpy(), vf.numpy()
    out["pre_o_causal"] = tg._gqa_prefill_ref(qf, kf, vf, heads=H, heads_kv=Hkv, is_causal=True).numpy()
    out["pre_o_full"] = tg._gqa_prefill_ref(qf, kf, vf, heads=H, heads_kv=Hkv, is_causal=False).numpy()
    out["pre_o_causal_softcap"] = tg._gqa_prefill_ref(
        qf, kf, vf, heads=H, heads_kv=Hkv, is_causal=True, softcap=2.0, sm_scale=0.125).numpy()
    out["pre_o_causal_bf16"] = bits(tg._gqa_prefill_ref(
        qf.bfloat16(), kf.bfloat16(), vf.bfloat16(), heads=H, heads_kv=Hkv, is_causal=True))
    ksq, vsq = kf[:, :Sq], vf[:, :Sq]
    out["pre_o_square"] = tg._gqa_prefill_ref(qf, ksq, vsq, heads=H, heads_kv=Hkv, is_causal=True).numpy()
    out["pre_lse_square"] = wl._compute_gqa_square_lse(
        qf, ksq, heads=H, heads_kv=Hkv, dim=D, is_causal=True).numpy()
    cu_q = torch.tensor([0, 24, 40], dtype=torch.int32)
    cu_k = torch.tensor([0, 50, 72], dtype=torch.int32)
    out["pre_o_varlen"] = tg._gqa_prefill_varlen_ref(
        qf[0], kf[0], vf[0], cu_q, cu_k, batch=2, heads=H, heads_kv=Hkv, is_causal=True).numpy()
    out["pre_cu_q"], out["pre_cu_k"] = cu_q.numpy(), cu_k.numpy()

    # ---- known-answer case of tests/ops/attention/test_gqa.py:417-443 (bottom-right mask)
    qa = torch.zeros(1, 128, 4, 64); ka = torch.zeros(1, 256, 2, 64); va = torch.zeros(1, 256, 2, 64)
    qa[..., 0] = 1; ka[..., 0] = 1; va[:, :128, :, 0] = 1; va[:, 128:, :, 0] = 100
    oa = tg._gqa_prefill_ref(qa, ka, va, heads=4, heads_kv=2, is_causal=True)
    out["kat_first"], out["kat_last"] = np.float32(oa[0, 0, 0, 0]), np.float32(oa[0, -1, 0, 0])

    # ---- FP8 quantiser: the reference function with pages playing the batch role
    P, page, Hkv, D = 6, 16, 2, 64
    xk = torch.randn(P, page, Hkv, D, generator=g).bfloat16()
    # fed as fp32 so that the scale is the fp32 ``amax / 448`` the FP8-cache decode workload asks for
    # (on a bf16 tensor the reference function would round the scale itself to bf16)
    xq, desc = fp8u.quantize_kv_fa3_descale(xk.float())
    out["fp8_x"] = bits(xk); out["fp8_q"] = bits(xq); out["fp8_scale"] = desc.numpy()
    # dequantise as tests/ops/attention/test_gqa_prefill_paged.py:355-356 (scale per page/head)
    out["fp8_dq_bf16"] = bits((xq.float() * desc[:, None, :, None]).to(torch.bfloat16))

    # ---- packed prefill over a paged cache with append (unaligned cached lengths, 16-token pages)
    from tests.ops.attention import test_gqa_prefill_paged as tpp
    q_lens, old_lens, H, Hkv, D, page, W = [17, 33], [37, 100], 4, 2, 32, 16, 10
    nb = len(q_lens)
    tq = sum(q_lens)
    cu = torch.tensor([0, 17, 50], dtype=torch.int32)
    bt = torch.randperm(nb * W, generator=g).to(torch.int32).reshape(nb, W)
    qn = torch.randn(tq, H, D, generator=g)
    kn = torch.randn(tq, Hkv, D, generator=g)
    vn = torch.randn(tq, Hkv, D, generator=g)
    k_old = [torch.randn(n, Hkv, D, generator=g) for n in old_lens]
    v_old = [torch.randn(n, Hkv, D, generator=g) for n in old_lens]
    kpg = torch.zeros(nb * W * page, Hkv, D)
    vpg = torch.zeros_like(kpg)
    tpp._fill_paged_cache_from_logical(kpg, vpg, k_old, v_old, bt, page)
    out["pp_q"], out["pp_k_new"], out["pp_v_new"] = qn.numpy(), kn.numpy(), vn.numpy()
    out["pp_k_pages"], out["pp_v_pages"] = kpg.numpy().copy(), vpg.numpy().copy()
    out["pp_cu"], out["pp_cache"], out["pp_bt"] = cu.numpy(), np.asarray(old_lens, np.int32), bt.numpy()
    out["pp_page"] = np.int32(page)
    kw = dict(batch=nb, heads=H, heads_kv=Hkv)
    out["pp_o_causal"] = tpp._gqa_prefill_paged_ref(qn, kn, vn, k_old, v_old, cu, is_causal=True, **kw).numpy()
    out["pp_o_full"] = tpp._gqa_prefill_paged_ref(qn, kn, vn, k_old, v_old, cu, is_causal=False, **kw).numpy()
    out["pp_o_softcap"] = tpp._gqa_prefill_paged_ref(qn, kn, vn, k_old, v_old, cu, is_causal=True,
                                                     softcap=2.0, **kw).numpy()
    out["pp_o_causal_f16"] = bits(tpp._gqa_prefill_paged_ref(
        qn.half(), kn.half(), vn.half(), [t.half() for t in k_old], [t.half() for t in v_old], cu,
        is_causal=True, **kw))
    # pages after the append, as the reference's test states it (test_gqa_prefill_paged.py:288-300)
    for b_, (ql, ol) in enumerate(zip(q_lens, old_lens)):
        for i in range(ql):
            pos = tpp._physical_pos(bt, b_, ol + i, page)
            kpg[pos] = kn[int(cu[b_]) + i]
            vpg[pos] = vn[int(cu[b_]) + i]
    out["pp_k_pages_after"], out["pp_v_pages_after"] = kpg.numpy(), vpg.numpy()

    # ---- sliding window: the reference tests' own reference programs, fixed length and packed
    from tests.ops.attention import test_gqa_sliding_window as tsw
    from tests.ops.attention import test_gqa_sliding_window_varlen as tswv
    B, S, H, Hkv, D = 2, 96, 4, 2, 32
    qs = torch.randn(B, S, H, D, generator=g)
    ks_ = torch.randn(B, S, Hkv, D, generator=g)
    vs_ = torch.randn(B, S, Hkv, D, generator=g)
    out["sw_q"], out["sw_k"], out["sw_v"] = qs.numpy(), ks_.numpy(), vs_.numpy()
    for name, (causal, wl, wr) in {"c_l17": (True, 17, -1), "n_l8_r5": (False, 8, 5), "n_r11": (False, -1, 11),
                                   "c_l0": (True, 0, -1)}.items():
        t = tsw.GroupedQueryAttentionSlidingWindowFwdTest(B, S, H, Hkv, D, causal, wl, wr, torch.float32)
        out["sw_o_" + name] = t.ref_program(qs, ks_, vs_).numpy()
    sq, sk = [24, 16], [50, 22]
    cuq = torch.tensor([0, 24, 40], dtype=torch.int32)
    cuk = torch.tensor([0, 50, 72], dtype=torch.int32)
    qv = torch.randn(40, H, D, generator=g)
    kv_ = torch.randn(72, Hkv, D, generator=g)
    vv_ = torch.randn(72, Hkv, D, generator=g)
    out["swv_q"], out["swv_k"], out["swv_v"] = qv.numpy(), kv_.numpy(), vv_.numpy()
    out["swv_cu_q"], out["swv_cu_k"] = cuq.numpy(), cuk.numpy()
    for name, (causal, wl, wr) in {"c_l9": (True, 9, -1), "n_l4_r6": (False, 4, 6)}.items():
        t = tswv.GroupedQueryAttentionSlidingWindowVarlenFwdTest(2, sq, sk, H, Hkv, D, causal, wl, wr, torch.float32)
        out["swv_o_" + name] = t.ref_program(qv, kv_, vv_, cuq, cuk, 24).numpy()

    # ---- NeoX RoPE at explicit positions: the reference test-suite's reference program and the
    # reference's own table generator (CPU)
    from tests.ops import test_rope as trp
    base_freqs = trp._compute_freqs_cis_base   # same formula as tileops.ops.rope.base_freqs (:97-120)
    xr = torch.randn(50, 3, 32, generator=g).half()
    pos = torch.cat([torch.arange(37, 37 + 17), torch.arange(100, 100 + 33)]).int()
    for name, rd in {"full": 32, "partial": 16}.items():
        cos, sin = base_freqs(rd, 134, dtype=torch.float16, device="cpu")
        out["rope_cos_" + name], out["rope_sin_" + name] = bits(cos), bits(sin)
        out["rope_y_" + name] = bits(trp.ref_rope_neox_position_ids(xr, cos, sin, pos.long(), rotary_dim=rd))
    out["rope_x"] = bits(xr)

    # ---- paged prefill over an FP8 cache with scalar scales: the expressions of the reference's test
    # (test_gqa_prefill_paged.py:348-404) around its reference program
    f8 = torch.float8_e4m3fn
    q_lens, old_lens, H, Hkv, D, page, W = [33, 48], [67, 80], 4, 2, 32, 16, 10
    cu = torch.tensor([0, 33, 81], dtype=torch.int32)
    bt = torch.randperm(2 * W, generator=g).to(torch.int32).reshape(2, W)
    ksc, vsc = torch.tensor([0.02]), torch.tensor([0.03])
    q8 = torch.randn(81, H, D, generator=g).half()
    kn8 = (torch.randn(81, Hkv, D, generator=g) * 0.5).half()
    vn8 = (torch.randn(81, Hkv, D, generator=g) * 0.5).half()
    k_old = [(torch.randn(n, Hkv, D, generator=g) * 0.5).half() for n in old_lens]
    v_old = [(torch.randn(n, Hkv, D, generator=g) * 0.5).half() for n in old_lens]
    k_old_q = [(t.float() / ksc[0]).to(f8) for t in k_old]
    v_old_q = [(t.float() / vsc[0]).to(f8) for t in v_old]
    kp8 = torch.zeros(2 * W * page, Hkv, D, dtype=f8)
    vp8 = torch.zeros_like(kp8)
    tpp._fill_paged_cache_from_logical(kp8, vp8, k_old_q, v_old_q, bt, page)
    k_old_dq = [(t.float() * ksc[0]).half() for t in k_old_q]
    v_old_dq = [(t.float() * vsc[0]).half() for t in v_old_q]
    out["p8_q"], out["p8_k_new"], out["p8_v_new"] = bits(q8), bits(kn8), bits(vn8)
    out["p8_k_pages"], out["p8_v_pages"] = bits(kp8), bits(vp8)
    out["p8_cu"], out["p8_cache"], out["p8_bt"] = cu.numpy(), np.asarray(old_lens, np.int32), bt.numpy()
    out["p8_page"], out["p8_k_scale"], out["p8_v_scale"] = np.int32(page), ksc.numpy(), vsc.numpy()
    out["p8_o"] = bits(tpp._gqa_prefill_paged_ref(q8, kn8, vn8, k_old_dq, v_old_dq, cu, batch=2, heads=H,
                                                   heads_kv=Hkv, is_causal=True))
    for b_, (ql, ol) in enumerate(zip(q_lens, old_lens)):
        for i in range(ql):
            pos = tpp._physical_pos(bt, b_, ol + i, page)
            kp8[pos] = (kn8[int(cu[b_]) + i].float() / ksc[0]).to(f8)
            vp8[pos] = (vn8[int(cu[b_]) + i].float() / vsc[0]).to(f8)
    out["p8_k_pages_after"], out["p8_v_pages_after"] = bits(kp8), bits(vp8)

    np.savez_compressed(os.path.join(HERE, "gqa_golden.npz"), **out)

    # ---- roofline formulas
    from tileops.perf import formulas as F
    roof = {
        "cfg1_decode": F.gqa_decode_roofline(q_shape=(2, 8, 64), kv_shape=(2, 256, 2, 64), dtype=torch.float32),
        "cfg2_fwd": F.gqa_fwd_roofline(q_shape=(4, 4096, 32, 128), kv_shape=(4, 4096, 8, 128),
                                       is_causal=True, dtype=torch.bfloat16),
        "fwd_noncausal_fp16": F.gqa_fwd_roofline(batch=2, seq_len=512, heads=64, heads_kv=8, dim=128,
                                                 is_causal=False, dtype=torch.float16),
        "decode_llama8b_4k": F.gqa_decode_roofline(q_shape=(32, 32, 128), kv_shape=(32, 4096, 8, 128),
                                                   dtype=torch.float16),
        "paged_probe": F.gqa_decode_paged_roofline(q_shape=(32, 32, 128), kv_shape=(4096, 8, 128),
                                                   page_size=64, dtype=torch.float16),
        "cfg4_paged_fp8": F.gqa_decode_paged_roofline(q_shape=(128, 64, 128), kv_shape=(524288, 8, 128),
                                                      page_size=64, dtype=torch.float8_e4m3fn),
        "cfg5_paged": F.gqa_decode_paged_roofline(q_shape=(8, 32, 128), kv_shape=(1048576, 8, 128),
                                                  page_size=128, dtype=torch.bfloat16),
        "varlen_packed": F.gqa_prefill_varlen_fwd_roofline(
            q_shape=(1024, 32, 128), k_shape=(8192, 8, 128), batch=2, max_seqlen_q=512,
            max_seqlen_kv=4096, q_lens=[512, 512], kv_lens=[4096, 4096], is_causal=True,
            dtype=torch.bfloat16),
        "varlen_ragged": F.gqa_prefill_varlen_fwd_roofline(
            q_shape=(40, 4, 32), k_shape=(72, 2, 32), batch=2, max_seqlen_q=24, max_seqlen_kv=50,
            q_lens=[24, 16], kv_lens=[50, 22], is_causal=True, dtype=torch.float16),
        "paged_prefill_llama8b": F.gqa_prefill_paged_with_kv_cache_fwd_roofline(
            total_q=4096, batch=8, q_lens=[512] * 8, cache_lens=[4096] * 8, heads=32, heads_kv=8, dim=128,
            page_size=64, max_pages_per_req=72, max_seqlen_q=512, is_causal=True, dtype=torch.float16),
        "paged_prefill_mixed": F.gqa_prefill_paged_with_kv_cache_fwd_roofline(
            total_q=4608, batch=8, q_lens=[256, 512, 768, 1024, 384, 640, 896, 128],
            cache_lens=[4096, 8192, 16384, 32768, 12288, 24576, 30720, 2048], heads=32, heads_kv=8, dim=128,
            page_size=64, max_pages_per_req=528, max_seqlen_q=1024, is_causal=True, dtype=torch.bfloat16),
        "paged_prefill_aggregate_only": F.gqa_prefill_paged_with_kv_cache_fwd_roofline(
            total_q=2048, batch=4, heads=8, heads_kv=2, dim=64, page_size=64, max_pages_per_req=72,
            max_seqlen_q=512, is_causal=False, dtype=torch.float16),
    }
    with open(os.path.join(HERE, "roofline_golden.json"), "w") as f:
        json.dump({k: list(map(int, v)) for k, v in roof.items()}, f, indent=1)
    print("wrote", os.path.join(HERE, "gqa_golden.npz"), os.path.getsize(os.path.join(HERE, "gqa_golden.npz")))


if __name__ == "__main__":
    main()
