"""SiLU-gated feed-forward: `down(silu(gate(x)) * up(x))`, no bias
(src/minillm/runtime.cpp:323-335; src/minillm/cuda/layer.cpp:65-70).

The gate and up matrices are stacked into one [2 I, width] operand at bind time,
so one product yields both; the kernel that applies the gate reads the two halves
of each row.  Parameters: hidden_size, intermediate_size.  Weights: "gate", "up"
[I, width], "down" [width, I].
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import register_part
from ..ops import functions as F
from ..weights.loader import WeightSpec
from .base import FeedForward, StepContext


class SwiGLU(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.width = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def weight_specs(self) -> List[WeightSpec]:
        w = self.spec.weights
        return [WeightSpec(w["gate"], (self.inter, self.width)), WeightSpec(w["up"], (self.inter, self.width)),
                WeightSpec(w["down"], (self.width, self.inter))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"] + (["gemm_f32"] if dtype is torch.float32 else ["gemm_bf16_tcgen05"])

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        self.w_gate_up = torch.cat([rt.matrix(tensors[w["gate"]]), rt.matrix(tensors[w["up"]])], dim=0).contiguous()
        self.w_down = rt.matrix(tensors[w["down"]])

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        rt = step.rt
        act = rt.gated_linear(x, self.w_gate_up)
        return rt.linear_delta(act, self.w_down, into=step.residual)


register_part("feed_forward", "swiglu", SwiGLU)
