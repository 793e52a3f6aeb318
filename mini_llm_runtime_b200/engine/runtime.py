"""The compute context parts share: device, precision, and the matrix product.

Two precisions exist.  `float32` is a true 32-bit path: weights, activations and the
cache are float32 and every matrix product runs on the package's own CUDA-core
kernel with float32 fused multiply-adds (no tensor cores, no TF32).  `bfloat16` is
the serving path: matrices, activations and the cache are bfloat16, products
accumulate in float32.  In both, the residual stream, norms, softmax, rotation and
logits are float32.

Which kernel a bfloat16 product takes depends on its rows and on what its result is; each
choice below is the faster one as measured in whole steps of the 8B sizes.
  * The gate/up product of a prompt portion of `pair_rows` rows or more runs on the package's
    two-SM tcgen05 kernel (`csrc/kernels/gemm_bf16_tcgen05_pair.cu`), which applies the SiLU
    gate in its epilogue: the product never goes to memory (the feed-forward keeps its two
    matrices interleaved in blocks of 128 rows for that).
  * With up to `decode_rows` rows, a product that ends a sub-layer (o_proj, down_proj) and the
    head run on the one-block tcgen05 kernel (`csrc/kernels/gemm_bf16_tcgen05.cu`): the
    weight matrix takes the 128-row side of the instruction, K is cut into ranges so that a
    small matrix still occupies every SM, and the kernel that reads the result adds the
    ranges' partial sums.
  * What is left goes to the vendor library (cuBLAS through `torch.mm` / `torch.addmm`), as the
    reference sends all of its products to cuBLAS (src/minillm/cuda/matrix.cpp:30-36): the
    few-row products whose result is an activation (q/k/v, gate/up), which the library writes
    in bfloat16 at once, and the plain products of prompt portions; one that ends a sub-layer
    adds its result into the residual stream in the library's epilogue.
`own_products_only()` takes the library out altogether: the two-SM kernel then runs every
product of 256 rows or more (adding into the residual stream in its own epilogue), the
one-block kernel the rest.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..ops import functions as F


class NonFiniteWeights(ValueError):
    """A tensor of the checkpoint holds a NaN or an infinity; the message names every such tensor."""


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
        self.use_tcgen05 = True       # bf16 products on the package's tcgen05/TMA kernel
        self.tcgen05_prefill = False  # the one-block kernel also for the row counts the vendor library takes by default
        # From this many rows on the gate/up product runs on the two-SM kernel with the gate in its
        # epilogue (against the library's product and a gate kernel it ties at 1024 rows and wins
        # beyond; in a 2048-token step of the 8B sizes it saves 4 % of the step).
        self.pair_rows = 1024
        self.pair_everything = False  # every product of 256 rows or more on the two-SM kernel
        self.tcgen05_attention = True  # prompt portions of 65 rows and more on the tcgen05 attention kernel
        # Up to this many rows a product runs on the own kernel (swapped operands, split K, partial
        # sums added by the kernel that reads them).  Measured in the decode step of the 8B sizes:
        # it wins by 5 % at 1 to 4 rows, ties at 8 and loses 3-4 % to the vendor library from 16
        # rows on, where its float32 partial sums (rows x splits) become real traffic.  64 is the
        # most the kernel's swapped form takes.
        self.decode_rows = 8
        # Of those few-row products, which ones: the two that end a sub-layer (o_proj,
        # down_proj: their split-K partial sums are added by the norm that follows, which adds
        # the residual anyway) and the head.  The two whose result is an activation (q/k/v,
        # gate/up) go to the vendor library unless this is set: its kernels write the bfloat16
        # result at once, and the decode step is 3-4 % faster that way at 1 to 8 rows.
        self.own_activation_products = False
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.pair_min_tiles = self.sm_count   # ... and only with at least this many 256 x 256 tiles
        self._splits = {}
        self._views = {}
        self._counters = None
        self._retired = []
        self.status = None        # the model's device status word (set at bind time)
        self._shared = {}
        self._load_names = None   # while weights are bound: id(source tensor) -> name, for the finiteness check
        self._load_flags = None
        self._load_checked = {}

    # ---- the finiteness check of uploaded weights
    def begin_load(self, tensors) -> None:
        """From here to `end_load`, every tensor of `tensors` that `matrix`, `vector` or
        `shared_matrix` uploads is checked on the device for NaNs and infinities, as the
        reference refuses such weights when it decodes them (src/minillm/cuda/storage.cpp:314-321).
        One flag per tensor, read once at the end."""
        self._load_names = {id(t): name for name, t in tensors.items()}
        self._load_flags = torch.zeros(max(1, len(tensors)), dtype=torch.int32, device=self.device)
        self._load_checked = {}

    def _checked(self, source: torch.Tensor, uploaded: torch.Tensor) -> torch.Tensor:
        name = self._load_names.get(id(source)) if self._load_names is not None else None
        if name is not None and name not in self._load_checked and uploaded.dtype in (torch.float32, torch.bfloat16):
            index = self._load_checked[name] = len(self._load_checked)
            F.finite_check(uploaded, self._load_flags[index:index + 1])
        return uploaded

    def end_load(self) -> None:
        names, flags = self._load_checked, self._load_flags
        self._load_names = self._load_flags = None
        self._load_checked = {}
        if names:
            bad = flags[:len(names)].cpu().tolist()
            broken = sorted(n for n, i in names.items() if bad[i])
            if broken:
                raise NonFiniteWeights(f"weights with non-finite values ({len(broken)}): " + ", ".join(broken))

    def own_products_only(self) -> None:
        """Every bfloat16 product on the package's tcgen05 kernels, none on the vendor library:
        few rows on the one-block kernel in its swapped form with split K (up to 64 rows) and
        in its plain form (up to `pair_rows`), more rows on the two-SM kernel as always.
        Slower than the default mix in decode steps (3 % at batch 8 of the 8B sizes); it
        shows that the package's kernels cover every product of the model."""
        self.decode_rows = 64
        self.own_activation_products = True
        self.tcgen05_prefill = True
        self.pair_everything = True
        self.pair_rows = 256

    @property
    def is_bf16(self) -> bool:
        return self.dtype is torch.bfloat16

    # ---- weights
    def matrix(self, t: torch.Tensor) -> torch.Tensor:
        """An operand of matrix products: the compute precision, on the device."""
        return self._checked(t, t.to(device=self.device, dtype=self.dtype).contiguous())

    def vector(self, t: torch.Tensor) -> torch.Tensor:
        """Norm weights and the like: float32 on the 32-bit path; on the bfloat16 path
        the stored precision is kept (a tensor stored in 32-bit stays 32-bit)."""
        if self.dtype is torch.float32:
            return self._checked(t, t.to(device=self.device, dtype=torch.float32).contiguous())
        return self._checked(t, t.to(device=self.device).contiguous())

    def shared_matrix(self, name: str, tensors) -> torch.Tensor:
        """A matrix several parts name (a tied embedding and head): one device copy."""
        if name not in self._shared:
            self._shared[name] = self.matrix(tensors[name])
        return self._shared[name]

    # ---- buffers
    def empty(self, *shape, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype or self.dtype, device=self.device)

    def split_counters(self, count: int) -> torch.Tensor:
        """Zeroed int32 counters for kernels that merge their own split results and leave the
        counters zero again.  One long-lived tensor, made outside any graph capture, so a
        captured step keeps pointing at it."""
        if self._counters is None or count > self._counters.numel():
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the split counters must be sized before a step is captured")
            if self._counters is not None:
                self._retired.append(self._counters)     # graphs captured earlier still point at it
            self._counters = torch.zeros(max(2 * count, 1 << 14), dtype=torch.int32, device=self.device)
        return self._counters

    # ---- y = x @ w.T
    def _transposed(self, w: torch.Tensor) -> torch.Tensor:
        """The view w.T the library takes, made once per weight matrix (an eager step calls
        for it some hundred times)."""
        view = self._views.get(id(w))
        if view is None or view[0] is not w:
            if len(self._views) >= 4096:      # someone multiplies by matrices that come and go: do not hold on to them
                self._views.clear()
            view = self._views[id(w)] = (w, w.t())
        return view[1]

    def _tcgen05_ok(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        return self.use_tcgen05 and self.status is not None and F.gemm_tcgen05_applies(x, w)

    def _pair(self, x: torch.Tensor, w: torch.Tensor, gated: bool = False) -> bool:
        """Whether this bf16 product runs on the two-SM kernel."""
        if not (gated or self.pair_everything) or x.shape[0] < self.pair_rows or not self._tcgen05_ok(x, w):
            return False
        # Fewer 256 x 256 tiles than SMs leave pairs idle (a small model's matrices); the library's
        # smaller tiles do better then.
        tiles = -(-x.shape[0] // 256) * -(-w.shape[0] // 256)
        return self.pair_everything or tiles >= self.pair_min_tiles

    def _own_gemm(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        """Whether this bf16 product runs on the one-block tcgen05 kernel: always for the few
        rows of a decode step; beyond those only when `tcgen05_prefill` is set."""
        return (x.shape[0] <= self.decode_rows or self.tcgen05_prefill) and self._tcgen05_ok(x, w)

    def linear(self, x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
               activation: bool = False) -> torch.Tensor:
        """x W^T.  `activation`: the result feeds a row-wise kernel as an activation (q/k/v,
        gate/up) rather than the residual stream or the logits."""
        out_dtype = out_dtype or self.dtype
        if self.dtype is torch.float32:
            out = torch.empty((x.shape[0], w.shape[0]), dtype=torch.float32, device=self.device)
            F.gemm_f32(x, w, out)
            return out
        if self._pair(x, w):
            out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=self.device)
            F.gemm_bf16_tcgen05_pair(x, w, out, self.status, "bf16" if out_dtype is torch.bfloat16 else "f32")
            return out
        if self._own_gemm(x, w) and (not activation or self.own_activation_products or self.tcgen05_prefill):
            out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=self.device)
            F.gemm_bf16_tcgen05(x, w, out, self.status)
            return out
        if out_dtype is torch.bfloat16:
            return torch.mm(x, self._transposed(w))
        return torch.mm(x, self._transposed(w), out_dtype=out_dtype)

    def linear_partials(self, x: torch.Tensor, w: torch.Tensor, activation: bool = False) -> Optional[torch.Tensor]:
        """For the few rows of a decode step: the product as float32 partial sums [S, M, N]
        over S ranges of K (so that a small weight matrix still occupies every SM); the
        kernel that reads them adds them up.  None when the product is not of that kind."""
        if self.dtype is not torch.bfloat16 or x.shape[0] > self.decode_rows or not self._own_gemm(x, w):
            return None
        if activation and not self.own_activation_products:
            return None
        key = (w.shape[0], w.shape[1])
        splits = self._splits.get(key)
        if splits is None:
            splits = self._splits[key] = F.k_splits_for(w.shape[0], w.shape[1], self.sm_count)
        out = torch.empty((splits, x.shape[0], w.shape[0]), dtype=torch.float32, device=self.device)
        F.gemm_bf16_tcgen05(x, w, out, self.status)
        return out

    def linear_delta(self, x: torch.Tensor, w: torch.Tensor, into: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
        """A float32 contribution to the residual stream: [M, N], or [S, M, N] partial sums
        that the next norm adds up.  With `into` (the stream itself, float32 [M, N]) the
        product of a prompt portion adds its result there in its epilogue (into += x W^T,
        one rounding per element as the separate add had) and None is returned."""
        parts = self.linear_partials(x, w)
        if parts is not None:
            return parts
        if into is not None and self.dtype is torch.bfloat16 and into.dtype is torch.float32 and into.is_contiguous():
            if self._pair(x, w):
                F.gemm_bf16_tcgen05_pair(x, w, into, self.status, "add_f32")
                return None
            if not self._own_gemm(x, w):
                torch.addmm(into, x, self._transposed(w), out_dtype=torch.float32, out=into)
                return None
        return self.linear(x, w, out_dtype=torch.float32)

    # ---- the gated pair of matrices of a feed-forward
    def stack_gate_up(self, w_gate: torch.Tensor, w_up: torch.Tensor):
        """The two [I, K] matrices as the one operand `gated_linear` takes, and the width I' of
        its result.  In bfloat16 the rows alternate in blocks of 128 (gate rows of 128 outputs,
        then their "up" rows), padded with zero rows to whole blocks, so that the gate can be
        applied in the epilogue of the product: I' = I rounded up to 128, and the extra
        outputs are zero.  In float32 all gate rows come first and I' = I."""
        w_gate, w_up = self.matrix(w_gate), self.matrix(w_up)
        if self.dtype is torch.bfloat16:
            stacked = F.interleave_gate_up(w_gate, w_up)
            return stacked, stacked.shape[0] // 2
        return torch.cat([w_gate, w_up], dim=0).contiguous(), w_gate.shape[0]

    def gated_linear(self, x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
        """silu(x Wgate^T) * (x Wup^T) for the operand `stack_gate_up` made."""
        inter = w_gate_up.shape[0] // 2
        block = F.GATE_BLOCK if self.dtype is torch.bfloat16 else inter
        out = torch.empty((x.shape[0], inter), dtype=self.dtype, device=self.device)
        if self.dtype is torch.bfloat16 and self._pair(x, w_gate_up, gated=True):
            F.gemm_bf16_tcgen05_pair(x, w_gate_up, out, self.status, "silu_gate")
            return out
        parts = self.linear_partials(x, w_gate_up, activation=True)
        F.swiglu(parts if parts is not None else self.linear(x, w_gate_up, activation=True), out, block)
        return out
