"""Weights by tensor name, from safetensors or from a seeded generator.

Element types kept on the device: with ``bfloat16`` as the run's type, 16-bit
floats become bfloat16 and a tensor stored in 32 bits stays float32; with
``float32`` every float becomes float32.  Integer tables become int32.

A checkpoint is checked as a whole before anything is copied: one
``WeightsError`` lists every missing tensor, every unexpected tensor and every
wrong shape (wlejon/brolm stops at the first missing name,
include/brolm/detail/weights.h:265-269, and checks the element count only,
:215-220).
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Iterable, Optional

import torch

from .safetensors_io import SafetensorsFile, iter_tensors, open_model_shards


class WeightsError(ValueError):
    def __init__(self, message: str, missing=(), unexpected=(), wrong_shape=()):
        super().__init__(message)
        self.missing, self.unexpected, self.wrong_shape = list(missing), list(unexpected), list(wrong_shape)


@dataclasses.dataclass
class Expected:
    shape: tuple
    role: str = "matrix"
    optional: bool = False


def kept_dtype(stored: torch.dtype, role: str, run_dtype: torch.dtype) -> torch.dtype:
    if role == "int" or not stored.is_floating_point:
        return torch.int32
    if run_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return run_dtype


def check_names(expected: dict[str, Expected], present: dict[str, tuple], where: str) -> None:
    """Raise one error that lists all that is wrong with a set of tensors."""
    missing = [n for n, e in expected.items() if n not in present and not e.optional]
    unexpected = [n for n in present if n not in expected]
    wrong = [(n, tuple(expected[n].shape), tuple(present[n])) for n in expected
             if n in present and tuple(present[n]) != tuple(expected[n].shape)]
    if not (missing or unexpected or wrong):
        return
    lines = [f"weights: {where} does not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(sorted(missing)))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + ", ".join(
            f"{n} is {list(got)}, expected {list(exp)}" for n, exp, got in sorted(wrong)))
    raise WeightsError("\n".join(lines), missing, unexpected, wrong)


def resolve_prefix(expected: dict[str, Expected], present: Iterable[str], prefix: str) -> dict[str, str]:
    """Map each expected name to the name the checkpoint uses: as written, or
    with ``prefix`` removed when the checkpoint was saved without that wrapper
    (wlejon/brolm src/gemma2.cpp:177-184)."""
    present = set(present)
    if not prefix:
        return {n: n for n in expected}
    with_prefix = sum(1 for n in expected if n.startswith(prefix) and n in present)
    bare = sum(1 for n in expected if n.startswith(prefix) and n[len(prefix):] in present)
    if bare > with_prefix:
        return {n: (n[len(prefix):] if n.startswith(prefix) else n) for n in expected}
    return {n: n for n in expected}


def load_from_folder(folder: str, expected: dict[str, Expected], run_dtype: torch.dtype, device,
                     optional_prefix: str = "") -> dict[str, torch.Tensor]:
    shards = open_model_shards(folder)
    where_is: dict[str, SafetensorsFile] = dict(iter_tensors(shards))
    names = resolve_prefix(expected, where_is.keys(), optional_prefix)
    expected_ckpt = {names[n]: e for n, e in expected.items()}
    check_names(expected_ckpt, {n: f.shape(n) for n, f in where_is.items()}, f"'{folder}'")
    out: dict[str, torch.Tensor] = {}
    for n, e in expected.items():
        ck = names[n]
        if ck not in where_is:
            continue
        t = where_is[ck].tensor(ck)
        out[n] = t.to(device=device, dtype=kept_dtype(t.dtype, e.role, run_dtype)).contiguous()
    return out


def load_from_tensors(tensors: dict[str, torch.Tensor], expected: dict[str, Expected], run_dtype: torch.dtype,
                      device, optional_prefix: str = "") -> dict[str, torch.Tensor]:
    names = resolve_prefix(expected, tensors.keys(), optional_prefix)
    expected_ckpt = {names[n]: e for n, e in expected.items()}
    check_names(expected_ckpt, {n: tuple(t.shape) for n, t in tensors.items()}, "the given tensors")
    out = {}
    for n, e in expected.items():
        t = tensors.get(names[n])
        if t is not None:
            out[n] = t.to(device=device, dtype=kept_dtype(t.dtype, e.role, run_dtype)).contiguous()
    return out
