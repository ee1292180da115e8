"""GPU peak profiles (role of ``src/tileops/perf/profile.py:69-84`` in the reference):
``load_profile(name)`` returns the YAML under ``perf/profiles/`` as a dict."""

from __future__ import annotations

import os

import yaml

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "profiles")


def available_profiles() -> list:
    return sorted(f[:-5] for f in os.listdir(_DIR) if f.endswith(".yaml"))


def load_profile(name: str) -> dict:
    path = os.path.join(_DIR, f"{name.lower()}.yaml")
    if not os.path.exists(path):
        raise FileNotFoundError(f"no GPU profile {name!r}; available: {available_profiles()}")
    with open(path) as fh:
        return yaml.safe_load(fh)
