"""Greedy and temperature sampling of the next token.

The reference chooses greedily only (argmax with ties to the lowest id,
src/minillm/cuda/ops.cu:166-201; its server rejects any other temperature,
src/http_server.cpp:140-142).  Temperature sampling is this engine's addition:
`softmax(logits / T)` inverted at a uniform number that is a pure function of
(seed, request, step), so a request draws the same tokens whatever else is in the
batch and however its prompt was cut.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from ..ops import functions as F

_MASK = (1 << 64) - 1


def uniform_for(seed: int, request: int, step: int) -> float:
    """A number in [0, 1) for the step-th draw of a request: the three integers are
    mixed by two rounds of a SplitMix64-style finaliser; the top 53 bits are used."""
    x = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB
         + 0x2545F4914F6CDD1D) & _MASK
    for _ in range(2):
        x ^= x >> 30
        x = (x * 0xBF58476D1CE4E5B9) & _MASK
        x ^= x >> 27
        x = (x * 0x94D049BB133111EB) & _MASK
        x ^= x >> 31
    return (x >> 11) / float(1 << 53)


@dataclass
class SamplingParams:
    max_tokens: int = 32
    temperature: float = 0.0
    seed: int = 0
    ignore_eos: bool = False

    def validate(self) -> None:
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        if not (self.temperature >= 0.0) or self.temperature == float("inf"):
            raise ValueError(f"temperature must be a finite number >= 0, got {self.temperature}")


class Sampler:
    """Samples one token per logits row on the device.  Temperatures and uniform numbers go to the device
    from two small pinned buffers (a ring of four, so a buffer is not written again while its copy may still
    be in flight), never from pageable memory."""
    _RING = 4

    def __init__(self, device, status: torch.Tensor, max_rows: int = 256):
        self.device = device
        self.status = status
        self._rows = 0
        self._turn = 0
        self._reserve(max_rows)

    def _reserve(self, rows: int) -> None:
        self._rows = rows
        self._host_t = [torch.empty(rows, dtype=torch.float32).pin_memory() for _ in range(self._RING)]
        self._host_u = [torch.empty(rows, dtype=torch.float64).pin_memory() for _ in range(self._RING)]
        self._done = [torch.cuda.Event() for _ in range(self._RING)]
        self._dev_t = torch.empty(rows, dtype=torch.float32, device=self.device)
        self._dev_u = torch.empty(rows, dtype=torch.float64, device=self.device)

    def sample(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
               uniforms: Optional[Sequence[float]] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 [rows] on the device (written to `out` when given); a row of non-finite logits gives -1."""
        rows = logits.shape[0]
        if out is None:
            out = torch.empty(rows, dtype=torch.int32, device=self.device)
        if temperatures is None or not any(t > 0 for t in temperatures):
            F.sample(logits, out, self.status)
            return out
        if rows > self._rows:
            torch.cuda.current_stream(self.device).synchronize()
            self._reserve(2 * rows)
        turn = self._turn
        self._turn = (turn + 1) % self._RING
        self._done[turn].synchronize()
        self._host_t[turn][:rows] = torch.tensor(list(temperatures), dtype=torch.float32)
        self._host_u[turn][:rows] = torch.tensor(list(uniforms), dtype=torch.float64)
        self._dev_t[:rows].copy_(self._host_t[turn][:rows], non_blocking=True)
        self._dev_u[:rows].copy_(self._host_u[turn][:rows], non_blocking=True)
        self._done[turn].record()
        F.sample(logits, out, self.status, self._dev_t[:rows], self._dev_u[:rows])
        return out
