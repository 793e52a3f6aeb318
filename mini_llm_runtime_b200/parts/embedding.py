"""Token embedding (a row gather, no scaling: src/minillm/runtime.cpp:224-228) and
the output head (`logits = x W^T` in float32: src/minillm/runtime.cpp:338-351).
When the head names the embedding's tensor the two share one device copy.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.registry import register_part
from ..ops import functions as F
from ..weights.loader import WeightSpec
from .base import Part, StepContext


class TokenEmbedding(Part):
    category = "embedding"

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(spec.params["vocab_size"])
        self.width = int(spec.params["width"])
        self.table = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["weight"], (self.vocab, self.width))]

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"]

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.table = rt.shared_matrix(self.spec.weights["weight"], tensors)

    def forward(self, step: StepContext) -> torch.Tensor:
        h = step.rt.empty(step.num_rows, self.width, dtype=torch.float32)
        F.embed_gather(self.table, step.token_ids, h, step.status)
        return h


class LinearHead(Part):
    category = "lm_head"

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(spec.params["vocab_size"])
        self.width = int(spec.params["width"])
        self.weight = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.spec.weights["weight"], (self.vocab, self.width))]

    def kernel_modules(self, dtype) -> List[str]:
        return F.product_modules(dtype)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        self.weight = rt.shared_matrix(self.spec.weights["weight"], tensors)

    def forward(self, x: torch.Tensor, step: StepContext) -> torch.Tensor:
        return step.rt.linear(x, self.weight, out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("lm_head", "linear_head", LinearHead)
