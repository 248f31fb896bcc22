"""What every part of a layer is: a named kind, parameters with declared
shapes, and a registry so that a layout can ask for a part by name.

Kinds: ``mixer`` (attention here), ``feedforward``, ``norm``, ``position`` and
``block`` (the arrangement of the others around the residual stream).
A part gets its sizes and constants as constructor arguments and never learns
which model it sits in; the checkpoint names of its tensors are given to it by
the layout, per instance.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional

import torch

KINDS = ("mixer", "feedforward", "norm", "position", "block")


@dataclasses.dataclass(frozen=True)
class ParamSpec:
    """One tensor a part needs.  ``role``: ``matrix`` (a projection, (out, in)),
    ``vector`` (a gain or bias), ``table`` (looked up by index), ``int`` (an
    integer table, kept as int32)."""
    shape: tuple
    role: str = "matrix"


class Part:
    """Base of all parts."""

    kind: str = ""
    # True when ``forward`` only launches work on the current stream, with
    # nothing that depends on values read back to the host: the decode step may
    # then be captured in a CUDA graph and replayed.
    graph_safe: bool = False

    def param_specs(self) -> dict[str, ParamSpec]:
        """Local tensor name -> what it must look like."""
        return {}

    def bind(self, params: dict[str, torch.Tensor]) -> None:
        """Take the loaded tensors (already on the device, in their kept
        element type).  A part may fuse or re-lay them out here."""
        self.params = params

    def cache_spec(self) -> Optional[Any]:
        """What the part keeps per sequence between steps (mixers only)."""
        return None

    def prepare(self, max_positions: int, device: torch.device) -> None:
        """Called when a cache is made: build tables that depend on its length."""


_REGISTRY: dict[str, dict[str, type]] = {k: {} for k in KINDS}


def register_part(kind: str, name: str, cls: type) -> None:
    """Make ``cls`` available to layouts as part ``name`` of ``kind``."""
    if kind not in _REGISTRY:
        raise ValueError(f"unknown part kind '{kind}' (kinds: {KINDS})")
    _REGISTRY[kind][name] = cls


def part_class(kind: str, name: str) -> type:
    try:
        return _REGISTRY[kind][name]
    except KeyError:
        raise KeyError(f"no {kind} part named '{name}' is registered "
                       f"(registered: {sorted(_REGISTRY.get(kind, {}))})") from None


def registered_parts(kind: str) -> list[str]:
    return sorted(_REGISTRY[kind])


@dataclasses.dataclass
class PartSpec:
    """A part as a layout writes it down: kind, registered name, constructor
    arguments, and the checkpoint name of each of its tensors."""
    kind: str
    name: str
    args: dict = dataclasses.field(default_factory=dict)
    tensors: dict = dataclasses.field(default_factory=dict)   # local name -> checkpoint name

    def build(self, **extra: Any) -> Part:
        part = part_class(self.kind, self.name)(**self.args, **extra)
        part.kind = self.kind
        return part
