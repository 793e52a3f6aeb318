"""SiLU-gated feed-forward: `down(silu(gate(x)) * up(x))`, no bias
(src/minillm/runtime.cpp:323-335; src/minillm/cuda/layer.cpp:65-70).

The gate and up matrices are stacked into one operand at bind time, so one product
yields both, and the gate is applied by that product's epilogue or by the kernel that
reads its result; how the rows are stacked is the runtime's business
(`Runtime.stack_gate_up`), which may round the inner width up (the extra activations
are zero, and "down" gets zero columns for them).  Parameters: hidden_size,
intermediate_size.  Weights: "gate", "up" [I, width], "down" [width, I].
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
        return ["elementwise"] + F.product_modules(dtype)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        self.w_gate_up, inner = rt.stack_gate_up(tensors[w["gate"]], tensors[w["up"]])
        self.w_down = rt.matrix(tensors[w["down"]])
        if inner != self.inter:
            padded = torch.zeros((self.width, inner), dtype=self.w_down.dtype, device=self.w_down.device)
            padded[:, :self.inter] = self.w_down
            self.w_down = padded

    def emit(self, b, x):
        act = b.rt.gated_linear(b, x, self.w_gate_up)
        return b.rt.linear_delta(b, act, self.w_down, into=b.residual)


register_part("feed_forward", "swiglu", SwiGLU)
