"""The compute context parts share: device, precision, and the matrix product.

Two precisions exist.  `float32` is a true 32-bit path: weights, activations and the
cache are float32 and every matrix product runs on the package's own CUDA-core
kernel with float32 fused multiply-adds (no tensor cores, no TF32).  `bfloat16` is
the serving path: matrices, activations and the cache are bfloat16, products
accumulate in float32.  In both, the residual stream, norms, softmax, rotation and
logits are float32.

Matrix products of the bfloat16 path go to the vendor library (cuBLAS through
`torch.mm`), as the reference sends all of its products to cuBLAS
(src/minillm/cuda/matrix.cpp:30-36), unless a hand-written kernel of this package
covers the shape: products for at most 16 tokens run on `csrc/kernels/gemv_bf16.cu`.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import functions as F


class Runtime:
    def __init__(self, dtype: torch.dtype = torch.bfloat16, device: str = "cuda:0"):
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"precision must be float32 or bfloat16, got {dtype}")
        if not torch.cuda.is_available():
            raise RuntimeError("mini-llm-runtime_b200 needs a CUDA GPU (sm_100a); there is no CPU path")
        self.dtype = dtype
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        # The 32-bit path must not be silently lowered by library defaults either.
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False
        self.use_gemv = False     # few-token products on the package's mma.sync weight streamer (slower than the library today)
        self.status = None        # the model's device status word (set at bind time)
        self._shared = {}

    @property
    def is_bf16(self) -> bool:
        return self.dtype is torch.bfloat16

    # ---- weights
    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """An operand of matrix products: the compute precision, on the device."""
        return t.to(device=self.device, dtype=self.dtype).contiguous()

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights and the like: float32 on the 32-bit path; on the bfloat16 path
        the stored precision is kept (a tensor stored in 32-bit stays 32-bit)."""
        if self.dtype is torch.float32:
            return t.to(device=self.device, dtype=torch.float32).contiguous()
        return t.to(device=self.device).contiguous()

    def shared_matrix(self, name: str, tensors) -> torch.Tensor:
        """A matrix several parts name (a tied embedding and head): one device copy."""
        if name not in self._shared:
            self._shared[name] = self.matrix(tensors[name])
        return self._shared[name]

    # ---- buffers
    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    # ---- y = x @ w.T
    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        out_dtype = out_dtype or self.dtype
        if self.dtype is torch.float32:
            out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=self.device)
            F.gemm_f32(x, w, out)
            return out
        if self.use_gemv and self.status is not None and F.gemv_applies(x, w):
            out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=self.device)
            F.gemv_bf16(x, w, out, self.status)
            return out
        if out_dtype is torch.bfloat16:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)

    def gated_linear(self, x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
        """silu(x Wgate^T) * (x Wup^T) for the stacked matrix [2 I, K]: one fused kernel for a
        few tokens, else the product followed by the gate kernel."""
        inter = w_gate_up.shape[0] // 2
        out = torch.empty((x.shape[0], inter), dtype=self.dtype, device=self.device)
        if self.dtype is torch.bfloat16 and self.use_gemv and self.status is not None and F.gemv_applies(x, w_gate_up):
            F.gemv_bf16(x, w_gate_up, out, self.status, swiglu=True)
            return out
        F.swiglu(self.linear(x, w_gate_up), out)
        return out
