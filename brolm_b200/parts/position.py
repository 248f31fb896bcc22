"""Position encodings."""
from __future__ import annotations

from typing import Optional

import torch

from .base import Part, register_part


class RotaryEmbedding(Part):
    """Rotation of the pairs (i, i + rot/2) of a head by pos * theta^(-2i/rot).

    Frequencies as wlejon/brolm states them (src/qwen35_text.cpp:220-256);
    the pairing is the checkpoint's, see csrc/core.cu.  The table of
    (cos, sin) is computed in float64 on the host and kept as float32, so the
    angles carry no rounding of their own.
    """

    kind = "position"

    def __init__(self, head_dim: int, theta: float, rotary_dim: Optional[int] = None):
        self.head_dim = head_dim
        self.theta = float(theta)
        self.rotary_dim = rotary_dim or head_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        self.table: Optional[torch.Tensor] = None
        self._outgrown: list = []      # earlier, shorter tables: a captured step may still read them

    def prepare(self, max_positions: int, device: torch.device) -> None:
        if self.table is not None and self.table.shape[0] >= max_positions and self.table.device == device:
            return
        if self.table is not None:
            # The part is shared by every layer and by every engine of its model; a CUDA graph that an
            # earlier engine captured holds the old table's address, so the old table is never freed.
            self._outgrown.append(self.table)
        half = self.rotary_dim // 2
        i = torch.arange(half, dtype=torch.float64)
        inv_freq = torch.tensor(self.theta, dtype=torch.float64) ** (-2.0 * i / self.rotary_dim)
        ang = torch.arange(max_positions, dtype=torch.float64)[:, None] * inv_freq[None, :]
        self.table = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.float32).contiguous().to(device)


register_part("position", "rope", RotaryEmbedding)
