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
from ..ops import native
from .base import Embedding, Head


class TokenEmbedding(Embedding):
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

    def emit(self, b):
        """h[r, :] = table[ids[r], :] as float32; an id outside the table zeroes the row and sets a status bit."""
        h = b.temp(b.rows, self.width, torch.float32)
        b.launch("elementwise", "mlr_embed_gather", h.ptr, self.table.data_ptr(), native.is_bf16(self.table), b.meta("token_ids"),
                 b.rows, self.width, self.vocab, b.status, b.stream)
        return h


class LinearHead(Head):
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

    def emit(self, b, x):
        return b.rt.linear(b, x, self.weight, out_dtype=torch.float32, out=b.logits(self.vocab))


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("lm_head", "linear_head", LinearHead)
