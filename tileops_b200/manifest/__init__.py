"""Loader of the operator specs (role of ``tileops.manifest``,
``src/tileops/manifest/__init__.py:41-96`` in the reference)."""

from __future__ import annotations

import functools
import os

import yaml

_DIR = os.path.dirname(os.path.abspath(__file__))

#: keys of a workload entry that are not op parameters
WORKLOAD_RESERVED_KEYS = frozenset({"dtypes", "label", "bench_skip_reason", "own_pages"})


@functools.lru_cache(maxsize=1)
def load_manifest() -> dict:
    """All op entries, keyed by op class name."""
    out: dict = {}
    for name in sorted(os.listdir(_DIR)):
        if name.endswith(".yaml"):
            with open(os.path.join(_DIR, name)) as fh:
                out.update(yaml.safe_load(fh) or {})
    return out


def load_workloads(op: str) -> list:
    """The ``workloads`` list of one op."""
    return list(load_manifest()[op].get("workloads", []))
