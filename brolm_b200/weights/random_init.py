"""Random weights from a configuration and a seed.

The values are a pure function of (seed, tensor name, element index), made of
integer arithmetic only, so the CPU and a GPU give the same bits: a model
that was filled on the device can be copied to the host and handed to
another implementation, and a tensor's values do not depend on which other
tensors exist or on the order they are made in.

    key      = first 8 bytes of sha256("<seed>:<name>")
    z_j      = splitmix64 output number 3 i + j + 1 of the stream that starts at key   (j = 0, 1, 2)
    s        = sum of the twelve 16-bit fields of z_0, z_1, z_2       (an integer below 2^20)
    value(i) = float32((s - 393210) / 65536) * std                     (one float32 rounding)

The sum of twelve uniform numbers has mean 6 and variance 1 (Irwin-Hall), so
value is N(0, std) to the eye, within +-6 std.  Matrices and tables use
``weight_std``, gain vectors ``norm_std``; the result is rounded once more to
the storage type.  wlejon/brolm has no such mode; its tests write a
uniform(-0.1, 0.1) fixture (tests/test_gemma2.cpp:97-106).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator

import torch

from .loader import Expected
from .safetensors_io import write_safetensors

_MASK64 = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_MIX1 = 0xBF58476D1CE4E5B9
_MIX2 = 0x94D049BB133111EB
CHUNK = 1 << 24          # elements drawn at a time (the temporaries are 64-bit)


def _signed(x: int) -> int:
    """The int64 with the bits of x mod 2^64 (torch has no unsigned 64-bit arithmetic)."""
    x &= _MASK64
    return x - (1 << 64) if x >> 63 else x


def _seed_of(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def _lsr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 (``>>`` keeps the sign)."""
    return (z >> n) & ((1 << (64 - n)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    """The output function of splitmix64 on int64 tensors (products wrap mod 2^64)."""
    z = (z ^ _lsr(z, 30)) * _signed(_MIX1)
    z = (z ^ _lsr(z, 27)) * _signed(_MIX2)
    return z ^ _lsr(z, 31)


def normal_values(key: int, start: int, count: int, std: float, device) -> torch.Tensor:
    """Elements [start, start + count) of the stream of ``key`` as float32 on ``device``."""
    i = torch.arange(start, start + count, dtype=torch.int64, device=device)
    total = torch.zeros(count, dtype=torch.int64, device=device)
    for j in range(3):
        z = _mix((i * 3 + (j + 1)) * _signed(_GOLDEN) + _signed(key))
        for shift in (0, 16, 32, 48):
            total += (z >> shift) & 0xFFFF
    centred = (total - 393210).to(torch.float32) / 65536.0        # exact: an integer below 2^24 over a power of two
    return centred * torch.tensor(std, dtype=torch.float32, device=device)


def random_tensor(seed: int, name: str, shape, std: float, dtype: torch.dtype, device) -> torch.Tensor:
    key = _seed_of(seed, name)
    n = 1
    for s in shape:
        n *= int(s)
    out = torch.empty(n, dtype=dtype, device=device)
    for start in range(0, n, CHUNK):
        count = min(CHUNK, n - start)
        out[start:start + count] = normal_values(key, start, count, std, device).to(dtype)
    return out.view(*shape)


def random_tensors(expected: dict[str, Expected], seed: int, weight_std: float, norm_std: float,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Iterator[tuple[str, torch.Tensor]]:
    """Yield (name, tensor) for every non-optional expected tensor, made on ``device``
    (the same values wherever they are made)."""
    device = torch.device(device)
    for name, e in expected.items():
        if e.optional:
            continue
        if e.role == "int":
            yield name, torch.zeros(e.shape, dtype=torch.int32, device=device)
            continue
        yield name, random_tensor(seed, name, e.shape, norm_std if e.role == "vector" else weight_std, dtype, device)


def write_model_folder(folder: str, config_dict: dict, expected: dict[str, Expected], seed: int,
                       weight_std: float, norm_std: float, dtype: torch.dtype = torch.bfloat16, device="cpu") -> None:
    """``device``: where the values are made before they are written (a GPU makes a large model in
    seconds; the file is the same)."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config_dict, fh, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      ((n, t.cpu()) for n, t in random_tensors(expected, seed, weight_std, norm_std, dtype, device)))
