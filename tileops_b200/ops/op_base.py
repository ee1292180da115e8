"""Operator base class: kernel-map install, kernel selection, get-or-build cache, target fork.

Behavioural mirror of the parts of ``tileops.ops.op_base.Op`` the GQA ops use
(``src/tileops/ops/op_base.py:53-656`` in the reference):

* ``dispatch_kernel(kernel_map)`` merges a caller's ``{slot: KernelClass}`` over the op's
  ``default_kernel_map`` and remembers which slots were replaced (``:196-222``);
* ``select_kernel_key(keys, call)`` picks the one implementation that serves a call:
  specialised beats ``general``, none / several / a refused replacement raise ``ValueError``
  with the reference's wording (``:238-301``);
* ``get_or_build_kernel`` caches one built kernel per key, and when a plugin target is
  settled, builds through the target's ``build_kernel(*TensorSpec, **manifest_params)`` keyed
  by device and input signature instead (``:311-425``);
* ``__call__`` settles the target once from ``target=``, the process default or the first
  tensor's device, and un-settles if that first call fails (``:557-618``);
* ``__init_subclass__`` installs ``_validate_dtypes``, ``eval_roofline`` and the manifest
  parameter names from the op's manifest entry (``:115-134``).

Constructing an op needs no device; only launching does.
"""

from __future__ import annotations

import re
from abc import ABC, abstractmethod
from types import MappingProxyType
from typing import Callable, Dict, Hashable, Iterator, Mapping, Optional, Sequence, Union

import torch

from ..backend.dispatch import registered_kernel_builder, registered_targets, select_target
from ..backend.errors import OpNotAvailableError
from ..backend.protocol import BUILTIN, Target, TensorSpec
from ..backend.registry import ensure_loaded
from ..kernels.kernel_base import Kernel
from ..manifest import load_manifest
from ..perf import formulas as _formulas

_UNRESOLVED = object()

_TORCH_DTYPES = {
    "float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32,
    "int32": torch.int32, "int64": torch.int64,
}
if hasattr(torch, "float8_e4m3fn"):
    _TORCH_DTYPES["float8_e4m3fn"] = torch.float8_e4m3fn


def _make_dtype_validator(op_name: str, inputs: Mapping[str, Mapping]) -> Callable:
    """Build ``_validate_dtypes(self, *tensors)`` from ``signature.inputs`` dtype rules
    (a union ``"a | b"`` or ``"same_as(x)"``); messages follow the reference's generated
    validator (``src/tileops/ops/_dtype_codegen.py:273-277``)."""
    names = list(inputs)
    rules = []
    for name in names:
        spec = str(inputs[name].get("dtype", ""))
        m = re.fullmatch(r"same_as\((\w+)\)", spec.strip())
        if m:
            rules.append(("same_as", m.group(1), spec))
        else:
            allowed = tuple(_TORCH_DTYPES[s.strip()] for s in spec.split("|") if s.strip() in _TORCH_DTYPES)
            rules.append(("union", allowed, spec))

    def _validate_dtypes(self, *tensors: torch.Tensor) -> None:
        if len(tensors) != len(names):
            raise ValueError(f"{op_name}: expected {len(names)} tensors ({', '.join(names)}), got {len(tensors)}")
        seen = dict(zip(names, tensors))
        for name, (kind, arg, spec) in zip(names, rules):
            t = seen[name]
            if t is None:
                continue
            if kind == "same_as":
                if t.dtype != seen[arg].dtype:
                    raise ValueError(f"{op_name}: input '{name}' has dtype {t.dtype}, expected '{spec}'")
            elif arg and t.dtype not in arg:
                raise ValueError(f"{op_name}: input '{name}' has dtype {t.dtype}, expected '{spec}'")

    return _validate_dtypes


class Op(ABC):
    """Base class of the operators."""

    target: Target = None
    _builder: object = _UNRESOLVED
    _settled_target: Target = None

    kernel_map: Optional[Dict[str, type]] = None
    _overridden_keys: frozenset = frozenset()
    dtype: Optional[torch.dtype] = None
    device: Optional[Union[torch.device, str]] = "cuda"
    tune: bool = False

    def __init_subclass__(cls, **kwargs: object) -> None:
        super().__init_subclass__(**kwargs)
        entry = load_manifest().get(cls.__name__)
        if entry is None:
            return
        sig = entry.get("signature", {})
        cls.__manifest_signature__ = sig
        cls.__manifest_param_names__ = tuple(sig.get("params") or {})
        if "_validate_dtypes" not in cls.__dict__:
            cls._validate_dtypes = _make_dtype_validator(cls.__name__, sig.get("inputs", {}))
        func = (entry.get("roofline") or {}).get("func")
        if func and "eval_roofline" not in cls.__dict__:
            fn = getattr(_formulas, func.rsplit(".", 1)[-1])

            def eval_roofline(self, _fn=fn):
                return _fn(self)

            cls.eval_roofline = eval_roofline

    # ---- kernel map ---------------------------------------------------------------------
    @property
    @abstractmethod
    def default_kernel_map(self) -> Dict[str, type]:
        raise NotImplementedError

    def _install_kernel_map(self, candidate_map: Optional[Dict[str, type]] = None) -> None:
        default_map = self.default_kernel_map
        override = dict(candidate_map) if candidate_map else {}
        if not default_map:
            self.kernel_map = override
            self._overridden_keys = frozenset(override)
            return
        self.kernel_map = {name: override.get(name, cls) for name, cls in default_map.items()}
        self._overridden_keys = frozenset(override) & frozenset(self.kernel_map)

    def dispatch_kernel(self, kernel_map: Optional[Dict[str, type]] = None) -> None:
        """Resolve and install the kernel map. Every op constructor ends here."""
        ensure_loaded()
        self._install_kernel_map(kernel_map)

    def select_kernel_key(self, keys: "tuple[str, ...]", call: object) -> str:
        """The one key among *keys* whose implementation serves *call*.

        When a plugin target has been settled for this instance the in-tree classes are not
        consulted at all (their architecture gate says nothing about another target's
        devices); the slot's last key names the role the target's kernel is cached under.
        The reference asks the in-tree classes first even then, which is why a stock install
        cannot reach a plugin on an architecture every in-tree class refuses.
        """
        if self._builder is not None and self._builder is not _UNRESOLVED:
            return keys[-1]
        applicable, rejected, refused = [], [], []
        for key in keys:
            kernel_cls = (self.kernel_map or {}).get(key)
            if kernel_cls is None:
                continue
            reason = kernel_cls.refusal(call)
            if reason is None:
                applicable.append(key)
                continue
            rejected.append(f"{key} ({kernel_cls.__name__}: {reason})")
            if key in self._overridden_keys:
                refused.append(f"{key} ({kernel_cls.__name__}: {reason})")
        specialised = [k for k in applicable if not self.kernel_map[k].general]
        chosen = specialised or applicable
        if len(chosen) == 1:
            if refused and chosen[0] not in self._overridden_keys:
                raise ValueError(
                    "the kernel supplied for " + "; ".join(refused)
                    + f" — selection does not fall back to the shipped '{chosen[0]}' "
                    f"when a replacement is in force. Call: {call}")
            return chosen[0]
        if not chosen:
            lead = ("the kernel supplied for " + "; ".join(refused) + ", and ") if refused else ""
            raise ValueError(
                lead + "no implementation serves this call: "
                + "; ".join(rejected or ["no implementation is installed"]) + f". Call: {call}")
        raise ValueError(
            f"dispatch is ambiguous: {', '.join(chosen)} all serve this call, so none is the answer. "
            f"Implementations of one key must serve disjoint regions, and at most one of them may "
            f"be general. Call: {call}")

    # ---- get-or-build ---------------------------------------------------------------------
    def get_or_build_kernel(self, name: str, inputs: "Sequence[torch.Tensor | None]", *,
                            key: Hashable = None, build: Optional[Callable[[], object]] = None):
        roles = getattr(self, "_kernel_roles", None)
        if roles is None:
            roles = {}
            self._kernel_roles = roles
        entries = roles.setdefault(name, {})
        settled_here = self._builder is _UNRESOLVED
        if settled_here:
            self._resolve_builder(tuple(inputs), {})
        try:
            builder = self._builder
            if builder is None or builder is _UNRESOLVED:
                if build is None:
                    raise OpNotAvailableError(
                        f"{type(self).__name__} has no in-tree implementation for {name!r}, so it "
                        f"needs a target that registers one; known targets for this op: "
                        f"{registered_targets(type(self).__name__)}")
                if key not in entries:
                    entries[key] = build()
                return entries[key]
            specs = tuple(None if t is None else TensorSpec.of(t) for t in inputs)
            present = tuple(s for s in specs if s is not None)
            if not present:
                raise OpNotAvailableError(
                    f"target {self._settled_target!r} serves {type(self).__name__}, but its "
                    f"{name!r} call site does not hand over the tensors a builder is described with")
            signature = (present[0].device,) + tuple(None if s is None else (s.dtype, s.shape) for s in specs)
            if signature not in entries:
                kernel = builder(*specs, **self._manifest_params())
                if not callable(kernel):
                    raise OpNotAvailableError(
                        f"target {self._settled_target!r} built {kernel!r} for "
                        f"{type(self).__name__}.{name}, which is not callable")
                entries[signature] = kernel
            return entries[signature]
        except Exception:
            if settled_here:
                self._unsettle()
            raise

    def _manifest_params(self) -> dict:
        values = {}
        for param in getattr(self, "__manifest_param_names__", ()) or ():
            try:
                values[param] = getattr(self, param)
            except AttributeError:
                raise AttributeError(
                    f"{type(self).__name__} declares manifest param {param!r} but keeps no "
                    f"attribute of that name") from None
        return values

    def built_kernels(self, role: str) -> Mapping[Hashable, object]:
        roles = getattr(self, "_kernel_roles", None) or {}
        return MappingProxyType(roles.get(role, {}))

    def iter_kernels(self) -> Iterator[Kernel]:
        seen = set()
        for entries in (getattr(self, "_kernel_roles", None) or {}).values():
            for entry in entries.values():
                if isinstance(entry, Kernel) and id(entry) not in seen:
                    seen.add(id(entry))
                    yield entry

    def autotune(self) -> None:
        """Tuned mode for what is held now and built later (the AOT kernels have fixed tunables)."""
        self.tune = True
        for kernel in self.iter_kernels():
            kernel.autotune()

    # ---- target settling ------------------------------------------------------------------
    @staticmethod
    def _first_tensor_device(args: tuple, kwargs: dict):
        for value in (*args, *kwargs.values()):
            if isinstance(value, torch.Tensor):
                return value.device
            if isinstance(value, (tuple, list)):
                for item in value:
                    if isinstance(item, torch.Tensor):
                        return item.device
        return None

    def _unsettle(self) -> None:
        self._builder = _UNRESOLVED
        self._settled_target = None
        self._kernel_roles = {}

    def _resolve_builder(self, args: tuple, kwargs: dict) -> None:
        device = self._first_tensor_device(args, kwargs)
        target = select_target(self.target, device)
        if target is None:
            self._settled_target = None
            if device is not None:
                self._builder = None
            return
        if target is BUILTIN:
            self._settled_target = BUILTIN
            self._builder = None
            return
        builder = registered_kernel_builder(type(self).__name__, target)
        if builder is None:
            raise OpNotAvailableError(
                f"target {target!r} registers no kernel builder for {type(self).__name__}; targets "
                f"that do: {registered_targets(type(self).__name__)}. There is no fall back to the "
                f"in-tree implementation: those kernels do not run on this target's devices.")
        self._settled_target = target
        self._builder = builder

    @abstractmethod
    def forward(self, *args: object, **kwargs: object):
        raise NotImplementedError

    def __call__(self, *args: object, **kwargs: object):
        if self._builder is not _UNRESOLVED:
            return self.forward(*args, **kwargs)
        self._resolve_builder(args, kwargs)
        try:
            return self.forward(*args, **kwargs)
        except Exception:
            self._unsettle()
            raise

    def eval_roofline(self) -> tuple:
        raise NotImplementedError(
            f"{type(self).__name__} has no manifest entry, so it has no roofline model")
