"""RMS norm, fused with the residual add that precedes it.

`(x * 1/sqrt(mean(x^2) + eps)) * w` over the full width, in float32
(src/minillm/kernels.cpp:209-216; GPU twin src/minillm/cuda/ops.cu:87-126).
Parameters: width, eps.  Weights: "weight" [width].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..ops import functions as F
from ..weights.loader import WeightSpec
from .base import Norm, StepContext


class RmsNorm(Norm):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["weight"], (self.width,), "vector", ("one_plus_normal", 0.01))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.weight = rt.vector(tensors[self.spec.weights["weight"]])

    def forward(self, h, delta, step: StepContext, rows=None):
        count = h.shape[0] if rows is None else rows.shape[0]
        out = step.rt.empty(count, self.width)
        F.rmsnorm(h, self.weight, self.eps, out, delta=delta, rows=rows, write_back=rows is None)
        return out


register_part("norm", "rmsnorm", RmsNorm)
