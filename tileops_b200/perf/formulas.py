"""Roofline work models ``(flops, bytes)`` of the GQA forward ops.

Numerically identical to the functions of the same names in the reference's
``tileops.perf.formulas`` (``src/tileops/perf/formulas.py:152-174, 478-529, 668-711``) so that
``op.eval_roofline()`` reports the same numbers on either implementation; the tests pin them
against values produced by the reference functions.  Each function accepts an op instance (its
attributes are read by name), a dict, or keyword arguments; ``q_shape``/``kv_shape`` take
precedence over scalar attributes.

Known quirk kept on purpose: the paged-decode flop count multiplies the POOL size by the
batch (every sequence is assumed to attend the whole pool).  For bandwidth or flop rates of a
batch whose sequences own disjoint pages use the workload's own byte/flop count instead
(``tileops_b200.workloads.PagedDecodeInputs.algorithmic_bytes``).
"""

from __future__ import annotations

from typing import Any

__all__ = [
    "gqa_fwd_roofline",
    "gqa_prefill_varlen_fwd_roofline",
    "gqa_prefill_paged_with_kv_cache_fwd_roofline",
    "gqa_decode_roofline",
    "gqa_decode_paged_roofline",
]


def _fields(op: Any, kwargs: dict) -> dict:
    if op is None:
        return kwargs
    return op if isinstance(op, dict) else vars(op)


def _itemsize(dtype: Any) -> int:
    if isinstance(dtype, (list, tuple)):
        dtype = dtype[0] if dtype else "float16"
    size = getattr(dtype, "itemsize", None)
    if size is not None:
        return int(size)
    name = str(dtype)
    for key, val in (("complex128", 16), ("complex64", 8), ("float32", 4), ("int32", 4),
                     ("float64", 8), ("int64", 8), ("bool", 1), ("int8", 1), ("uint8", 1)):
        if key in name:
            return val
    return 2


def _dtype_of(data: dict) -> Any:
    return data.get("dtype", data.get("dtypes", "float16"))


def gqa_fwd_roofline(op: Any = None, **kwargs: Any) -> tuple:
    """Dense GQA prefill: ``4*B*H*S^2*D`` flops (halved when causal); q, o, k, v once each."""
    d = _fields(op, kwargs)
    if "q_shape" in d:
        batch, seq_len, heads, dim = d["q_shape"]
        heads_kv = d["kv_shape"][2]
    else:
        batch, seq_len, heads, heads_kv, dim = (d[k] for k in ("batch", "seq_len", "heads", "heads_kv", "dim"))
    flops = 4 * batch * heads * seq_len * seq_len * dim
    if bool(d.get("is_causal", True)):
        flops //= 2
    q_elems = batch * seq_len * heads * dim
    kv_elems = batch * seq_len * heads_kv * dim
    return int(flops), int(2 * (q_elems + kv_elems) * _itemsize(_dtype_of(d)))


def _visible_scores(len_q: int, len_kv: int) -> int:
    # bottom-right aligned causal mask: only the last min(len_q, len_kv) query rows see keys
    rows = min(len_q, len_kv)
    return rows * len_kv - rows * (rows - 1) // 2


def _spread(total: int, batch: int, max_len: int) -> list:
    out, left = [0] * batch, total
    for i in range(batch):
        out[i] = min(max_len, left - (batch - i - 1))
        left -= out[i]
    return out


def gqa_prefill_varlen_fwd_roofline(op: Any = None, **kwargs: Any) -> tuple:
    """Packed (THD) GQA prefill with per-request lengths."""
    d = _fields(op, kwargs)
    if "q_shape" not in d and d.get("_roofline_kwargs") is not None:
        d = dict(d["_roofline_kwargs"])
    total_q, heads, dim = d["q_shape"]
    total_kv, heads_kv, _ = d["k_shape"]
    batch = int(d["batch"])
    q_lens, kv_lens = d.get("q_lens"), d.get("kv_lens")

    def from_cu(cu):
        vals = [int(x) for x in cu.detach().cpu().tolist()]
        return [b - a for a, b in zip(vals[:-1], vals[1:])]

    if q_lens is None and d.get("cu_seqlens_q") is not None:
        q_lens = from_cu(d["cu_seqlens_q"])
    if kv_lens is None and d.get("cu_seqlens_kv") is not None:
        kv_lens = from_cu(d["cu_seqlens_kv"])
    if q_lens is None:
        q_lens = _spread(total_q, batch, int(d["max_seqlen_q"]))
    if kv_lens is None:
        kv_lens = _spread(total_kv, batch, int(d["max_seqlen_kv"]))
    causal = bool(d.get("is_causal", True))
    if len(q_lens) != len(kv_lens):
        raise ValueError("q_lens and kv_lens differ in length")
    visible = sum(_visible_scores(int(a), int(b)) if causal else int(a) * int(b)
                  for a, b in zip(q_lens, kv_lens))
    e = _itemsize(_dtype_of(d))
    q_elems = total_q * heads * dim
    kv_elems = total_kv * heads_kv * dim
    return int(4 * heads * visible * dim), int((2 * q_elems + 2 * kv_elems) * e + 2 * (batch + 1) * 4)


def gqa_prefill_paged_with_kv_cache_fwd_roofline(op: Any = None, **kwargs: Any) -> tuple:
    """Packed prefill over a paged cache with append: every query row sees its request's cached
    tokens plus the causal part of the chunk; bytes = q, o, cached K/V read, new K/V read and
    written once more (the append), plus the int32 metadata.  Missing per-request lengths are
    filled deterministically from the aggregate fields, as the reference's formula does
    (``src/tileops/perf/formulas.py:532-587``)."""
    d = _fields(op, kwargs)
    batch, heads, heads_kv, dim = (int(d[k]) for k in ("batch", "heads", "heads_kv", "dim"))
    pages, page = int(d["max_pages_per_req"]), int(d["page_size"])
    max_q = int(d.get("max_seqlen_q", pages * page))
    causal = bool(d.get("is_causal", True))
    q_lens = d.get("q_lens")
    total_q = int(d["total_q"]) if "total_q" in d else (int(sum(q_lens)) if q_lens is not None else batch * max_q)
    if q_lens is None:
        q_lens = _spread(total_q, batch, max_q)
    cache_lens = d.get("cache_lens")
    if cache_lens is None:
        cap = pages * page if d.get("max_position") is None else int(d["max_position"])
        cache_lens = [max(cap - int(n), 0) for n in q_lens]
    if len(q_lens) != len(cache_lens):
        raise ValueError("q_lens and cache_lens differ in length")
    visible, cached = 0, 0
    for n, old in zip(q_lens, cache_lens):
        n, old = int(n), int(old)
        cached += old
        visible += n * old + n * (n + 1) // 2 if causal else n * (old + n)
    e = _itemsize(_dtype_of(d))
    q_elems = total_q * heads * dim
    new_kv = 2 * total_q * heads_kv * dim
    elems = 2 * q_elems + 2 * cached * heads_kv * dim + 2 * new_kv
    meta = (batch + 1) * 4 + batch * 4 + batch * pages * 4
    return int(4 * heads * visible * dim), int(elems * e + meta)


def gqa_decode_roofline(op: Any = None, **kwargs: Any) -> tuple:
    """Contiguous-cache decode."""
    d = _fields(op, kwargs)
    if "q_shape" in d:
        batch, heads, dim = d["q_shape"]
        _, seqlen_kv, heads_kv, _ = d["kv_shape"]
    else:
        batch, heads, heads_kv, seqlen_kv, dim = (d[k] for k in ("batch", "heads", "heads_kv", "seqlen_kv", "dim"))
    e = _itemsize(_dtype_of(d))
    q_elems = batch * heads * dim
    kv_elems = batch * seqlen_kv * heads_kv * dim
    return int(4 * batch * heads * seqlen_kv * dim), int((2 * q_elems + 2 * kv_elems) * e)


def gqa_decode_paged_roofline(op: Any = None, **kwargs: Any) -> tuple:
    """Paged-cache decode; ``seqlen_kv`` is the pool size in tokens."""
    d = _fields(op, kwargs)
    if "q_shape" in d:
        batch, heads, dim = d["q_shape"]
        seqlen_kv, heads_kv, _ = d["kv_shape"]
    else:
        batch, heads, heads_kv, seqlen_kv, dim = (d[k] for k in ("batch", "heads", "heads_kv", "seqlen_kv", "dim"))
    e = _itemsize(_dtype_of(d))
    page = int(d["page_size"])
    q_elems = batch * heads * dim
    kv_elems = seqlen_kv * heads_kv * dim
    meta = batch * 4 + batch * max(1, -(-seqlen_kv // page)) * 4
    return int(4 * batch * heads * seqlen_kv * dim), int((2 * q_elems + 2 * kv_elems) * e + meta)
