"""Rotary position encoding as a table of cosines and sines.

`freq_j = theta^(-2j/D)`, `angle = float(position) * freq_j`, all in float32, as
src/minillm/runtime.cpp:231-241 computes them for each step and
src/minillm/cuda/storage.cpp:261-287 tabulates them once ([positions, D], cosines
in the first half of a row, sines in the second).  The table is made on the host
with float32 `pow`, multiply, `cos` and `sin`, then uploaded; the mixer's kernel
rotates `(x[j], x[j + D/2])` pairs with it.
Parameters: theta, rotary_dim, max_positions.  No weights.
"""
from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..config.registry import register_part
from .base import PositionEncoding


def rotation_table(theta: float, rotary_dim: int, max_positions: int) -> torch.Tensor:
    half = rotary_dim // 2
    j = np.arange(half, dtype=np.float32)
    exponent = (np.float32(-2.0) * j / np.float32(rotary_dim)).astype(np.float32)
    freq = np.power(np.float32(theta), exponent).astype(np.float32)
    pos = np.arange(max_positions, dtype=np.float32)[:, None]
    angle = (pos * freq[None, :]).astype(np.float32)
    table = np.concatenate([np.cos(angle), np.sin(angle)], axis=1).astype(np.float32)
    return torch.from_numpy(table)


class Rope(PositionEncoding):
    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(spec.params["theta"])
        self.rotary_dim = int(spec.params["rotary_dim"])
        self.max_positions = int(spec.params["max_positions"])
        if self.rotary_dim % 2:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even")
        self._table: Optional[torch.Tensor] = None

    def bind(self, tensors, rt) -> None:
        self._table = rotation_table(self.theta, self.rotary_dim, self.max_positions).to(rt.device)

    def rotation_table(self) -> Optional[torch.Tensor]:
        return self._table


register_part("position", "rope", Rope)
