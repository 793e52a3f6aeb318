"""RMS norm, fused with the residual add that precedes it.

`(x * 1/sqrt(mean(x^2) + eps)) * w` over the full width, in float32
(src/minillm/kernels.cpp:209-216; GPU twin src/minillm/cuda/ops.cu:87-126).
Parameters: width, eps.  Weights: "weight" [width].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import register_part
from ..engine.builder import Buf
from ..ops import native
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

    def foldable(self):
        return ("rms", self.weight, self.eps, self.width)

    def emit(self, b, h, delta, wanted_only: bool = False):
        """out[r] = rmsnorm(h[row] + delta[row]) * weight, row = the r-th wanted row or r; unless only
        the wanted rows are normed, the sum is stored back to h, which moves the residual stream on.
        `delta` may be partial sums [S, M, width], which are added in order first."""
        count = b.want if wanted_only else h.rows
        prepared, b.prepared = b.prepared, None
        if delta is None and b.rt.norm_can_wait(b, count, self.width):
            # The product that reads this norm's result will norm its own input (a few-row product
            # streams the weights once and has the rows in shared memory anyway): nothing to launch here.
            # The product that last added into the stream may have left this norm half done.
            if prepared is not None and (wanted_only or prepared["stream"] != h.ptr or prepared["weight"] is not self.weight):
                prepared = None
            return Buf(None, count, self.width, b.rt.dtype, self.width, norm=(h, self.weight, self.eps, wanted_only, prepared))
        out = b.temp(count, self.width, b.rt.dtype)
        slices, stride = (delta.slices or 1, delta.slice_stride) if delta is not None else (1, 0)
        b.launch("elementwise", "mlr_rmsnorm", h.ptr, delta.ptr if delta is not None else None, slices, stride,
                 self.weight.data_ptr(), native.is_bf16(self.weight), out.ptr, out.is_bf16,
                 b.meta("want_rows") if wanted_only else None, count, self.width, self.eps, int(not wanted_only), b.stream,
                 need="want" if wanted_only else None)
        return out


register_part("norm", "rmsnorm", RmsNorm)
