"""Random weights from a configuration and a seed.

Every tensor draws from a generator of its own, seeded by (seed, tensor
name), so a tensor's values do not depend on which other tensors exist or on
the order they are made in.  Matrices and tables are N(0, weight_std), gain
vectors N(0, norm_std); values are rounded to the storage type.
wlejon/brolm has no such mode; its tests write a uniform(-0.1, 0.1) fixture
(tests/test_gemma2.cpp:97-106).
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Iterator

import torch

from .loader import Expected
from .safetensors_io import write_safetensors


def _seed_of(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & (2 ** 63 - 1)


def random_tensors(expected: dict[str, Expected], seed: int, weight_std: float, norm_std: float,
                   dtype: torch.dtype = torch.bfloat16, device="cpu") -> Iterator[tuple[str, torch.Tensor]]:
    """Yield (name, tensor) for every non-optional expected tensor.

    ``device='cpu'`` gives the same values on every machine; a CUDA device
    draws there (another stream of numbers, for large models in a hurry).
    """
    device = torch.device(device)
    for name, e in expected.items():
        if e.optional:
            continue
        gen = torch.Generator(device=device)
        gen.manual_seed(_seed_of(seed, name))
        if e.role == "int":
            yield name, torch.zeros(e.shape, dtype=torch.int32, device=device)
            continue
        std = norm_std if e.role == "vector" else weight_std
        t = torch.randn(e.shape, generator=gen, dtype=torch.float32, device=device) * std
        yield name, t.to(dtype)


def write_model_folder(folder: str, config_dict: dict, expected: dict[str, Expected], seed: int,
                       weight_std: float, norm_std: float, dtype: torch.dtype = torch.bfloat16) -> None:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as fh:
        json.dump(config_dict, fh, indent=1)
    write_safetensors(os.path.join(folder, "model.safetensors"),
                      random_tensors(expected, seed, weight_std, norm_std, dtype))
