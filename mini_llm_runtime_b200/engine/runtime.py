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
from ..ops import native
from . import executor
from .builder import Buf


class NonFiniteWeights(ValueError):
    """A tensor of the checkpoint holds a NaN or an infinity; the message names every such tensor."""


_library_workspace = {}     # device index -> the vendor library's workspace there (kept for the life of the process)


def _give_library_workspace(device: torch.device) -> None:
    """The vendor library gets 32 MiB of workspace from this package once per device, so that it
    allocates none of its own: a CUDA graph capture would not allow that, and a step in the steady
    state is to allocate nothing."""
    index = device.index or 0
    if index not in _library_workspace:
        space = torch.empty(32 << 20, dtype=torch.uint8, device=device)
        with torch.cuda.device(device):
            if executor.library().mlr_library_set_workspace(space.data_ptr(), space.numel()) != 0:
                raise RuntimeError(executor.library().mlr_exec_error().decode())
        _library_workspace[index] = space


_ROUTING = {"gemv_rows", "gemv_balance", "fuse_rotation_rows", "use_tcgen05", "tcgen05_prefill", "pair_rows", "pair_everything", "tcgen05_attention", "decode_rows",
            "own_activation_products", "pair_min_tiles"}


def units_balance(rows: int, sm_count: int) -> float:
    """How full the rounds are when `rows` rows of a matrix are dealt 16 at a time to one block per SM (1.0 when all
    units fit one round: then the SMs that get none are idle, but no block waits for another round)."""
    units = -(-rows // 16)
    if units <= sm_count:
        return 1.0
    return units / (-(-units // sm_count) * sm_count)


class Runtime:
    def __setattr__(self, name, value):
        # A change of a routing setting outdates the programs recorded with the old one.
        if name in _ROUTING:
            object.__setattr__(self, "routing_version", getattr(self, "routing_version", 0) + 1)
        object.__setattr__(self, name, value)

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
        # Up to this many rows (at most 8) a product is one pass over the weights by `gemv_bf16.cu`, with the norm
        # before it and the gate or the residual add after it folded in: a decode layer is then six launches
        # instead of nine and the vendor library is off the decode path.  In the decode step of the 8B sizes
        # (8 layers, context 2000, CUDA events) a step takes 0.887 ms at one request and 0.994 ms at eight that
        # way, against 1.013 and 1.087 ms with the split-K tcgen05 products, the library's q/k/v and gate/up and
        # the three row-wise kernels between them (0 switches back to those).
        self.gemv_rows = 8
        self.gemv_balance = 0.8
        # A step of decoded tokens only, of at most this many rows: the split-KV attention kernel norms, rotates and
        # writes the cache itself (no row-wise kernel between the q/k/v product and attention).  Measured in the decode
        # step of the 8B sizes (8 layers, context 2000): 0.867 ms against 0.884 ms at one request, 1.169 against 1.187 ms
        # at 16, but 1.700 against 1.660 ms at 64, where every one of many more blocks repeats the work on its queries.
        self.fuse_rotation_rows = 32
        self.sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.shared_memory_limit = torch.cuda.get_device_properties(self.device).shared_memory_per_block_optin
        if dtype is torch.bfloat16:
            _give_library_workspace(self.device)
        self.pair_min_tiles = self.sm_count   # ... and only with at least this many 256 x 256 tiles
        self._splits = {}
        self._gemv_fit = {}
        self._counters = None
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
        counters zero again (steps that Python drives; the native executor has its own)."""
        if self._counters is None or count > self._counters.numel():
            self._counters = torch.zeros(max(2 * count, 1 << 14), dtype=torch.int32, device=self.device)
        return self._counters

    # ---- y = x @ w.T, described to a builder (engine/builder.py)
    # `b` is the builder of the step (eager) or of the program being recorded; `x` a Buf of it; `w` a
    # weight tensor [N, K] on the device.  Every decision on a row count goes through `b.le` /
    # `b.ge`, so that a recorded program knows for which row counts it holds.
    def _tcgen05_ok(self, x: Buf, w: torch.Tensor) -> bool:
        K = w.shape[1]
        return (self.use_tcgen05 and x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and K % 8 == 0 and K >= 8
                and x.width == K and w.stride(1) == 1 and x.ld % 8 == 0 and w.stride(0) % 8 == 0 and x.ptr % 16 == 0
                and w.data_ptr() % 16 == 0)

    def _pair(self, b, x: Buf, w: torch.Tensor, gated: bool = False) -> bool:
        """Whether this bf16 product runs on the two-SM kernel: from `pair_rows` rows on, and only
        with at least `pair_min_tiles` tiles of 256 x 256 (fewer leave pairs of SMs idle: a small
        model's matrices; the library's smaller tiles do better then)."""
        if not (gated or self.pair_everything) or not self._tcgen05_ok(x, w):
            return False
        first = self.pair_rows
        if not self.pair_everything:
            across = -(-w.shape[0] // 256)
            first = max(first, 256 * (-(-self.pair_min_tiles // across) - 1) + 1)
        return b.ge(x.rows, first)

    def _own_gemm(self, b, x: Buf, w: torch.Tensor) -> bool:
        """Whether this bf16 product runs on the one-block tcgen05 kernel: always for the few
        rows of a decode step; beyond those only when `tcgen05_prefill` is set."""
        return self._tcgen05_ok(x, w) and (self.tcgen05_prefill or b.le(x.rows, self.decode_rows))

    def _own_launch(self, b, x: Buf, w: torch.Tensor, out: Buf) -> None:
        """The one-block tcgen05 product into `out` (bf16, float32, or float32 partial sums).  With up
        to 64 rows the weight matrix takes the 128-row side of the instruction and the result is
        stored transposed; otherwise x takes that side.  `w` must hold weights: the kernel starts to
        fetch it before the kernels before it on the stream are done."""
        N, K = w.shape
        splits, stride = max(1, out.slices), out.slice_stride
        f32 = int(out.dtype is torch.float32)
        if b.le(x.rows, 64):
            b.launch("gemm_bf16_tcgen05", "mlr_gemm_bf16_tcgen05", w.data_ptr(), w.stride(0), N, x.ptr, x.ld, x.rows, K, out.ptr,
                     out.ld, f32, 1, 0, splits, stride, 1, b.status, b.stream, need=b.need_for(x.rows))
        else:
            b.launch("gemm_bf16_tcgen05", "mlr_gemm_bf16_tcgen05", x.ptr, x.ld, x.rows, w.data_ptr(), w.stride(0), N, K, out.ptr,
                     out.ld, f32, 0, 0, splits, stride, 2, b.status, b.stream, need=b.need_for(x.rows))

    def _pair_launch(self, b, x: Buf, w: torch.Tensor, out: Buf, epilogue: str) -> None:
        b.launch("gemm_bf16_tcgen05_pair", "mlr_gemm_bf16_tcgen05_pair", x.ptr, x.ld, x.rows, w.data_ptr(), w.stride(0), w.shape[0],
                 w.shape[1], out.ptr, out.ld, F.PAIR_EPILOGUES[epilogue], b.status, b.stream, need=b.need_for(x.rows))

    def _library_launch(self, b, x: Buf, w: torch.Tensor, out: Buf, accumulate: bool = False) -> None:
        """The vendor library's product (cuBLAS), as the reference sends all of its products there
        (src/minillm/cuda/matrix.cpp:30-36)."""
        b.launch("host", "mlr_library_gemm", x.ptr, x.ld, x.rows, w.data_ptr(), w.stride(0), w.shape[0], w.shape[1], out.ptr,
                 out.ld, int(out.dtype is torch.float32), int(accumulate), b.stream, need=b.need_for(x.rows))

    # ---- few rows: a pass over the weights with the neighbouring row-wise work folded in
    def _gemv_fits(self, K: int, adds: bool = False) -> bool:
        """Whether the few-row kernel takes `gemv_rows` rows of K values (a product that adds into the stream is cut
        along K until it does)."""
        key = (min(self.gemv_rows, 8), K, adds)
        if key not in self._gemv_fit:
            self._gemv_fit[key] = K % 8 == 0 and (adds or bool(native.module("gemv_bf16").mlr_gemv_bf16_fits(key[0], K)))
        return self._gemv_fit[key]

    def norm_can_wait(self, b, count, width: int) -> bool:
        """Whether a norm over `count` rows of `width` need not be launched because the product that
        reads it will do it in its prologue."""
        return self.dtype is torch.bfloat16 and self.gemv_rows > 0 and self._gemv_fits(width) and b.le(count, min(self.gemv_rows, 8))

    def _gemv(self, b, x: Buf, w: torch.Tensor, adds: bool = False) -> bool:
        """Whether this bf16 product (`adds`: into the float32 stream) is a few-row pass over the weights."""
        if (self.dtype is not torch.bfloat16 or self.gemv_rows <= 0 or w.dtype is not torch.bfloat16
                or not self._gemv_fits(w.shape[1], adds and x.norm is None)):
            return False
        if w.stride(1) != 1 or w.stride(0) % 8 or w.data_ptr() % 16 or x.width != w.shape[1]:
            return False
        # The kernel deals 16 rows of W at a time to one block per SM: a matrix whose units leave the last round
        # mostly empty (320 units over 148 SMs: 2.2 rounds cost 3) is better off with K cut across the SMs.
        if units_balance(w.shape[0], self.sm_count) < self.gemv_balance:
            return False
        if x.norm is None and (x.dtype is not torch.bfloat16 or x.ld % 8 or x.ptr % 16):
            return False
        return b.le(x.rows, min(self.gemv_rows, 8))

    def _gemv_launch(self, b, x: Buf, w: torch.Tensor, out: Buf, mode: str) -> None:
        N, K = w.shape
        ahead = None
        if mode == "add_f32":
            ahead, b.norm_ahead = b.norm_ahead, None
        if x.norm is not None and x.norm[4] is not None:
            # The product that added into the stream last left this norm half done.
            prepared = x.norm[4]
            b.launch("gemv_bf16", "mlr_gemv_bf16_prepared", w.data_ptr(), w.stride(0), N, K, prepared["side"].ptr, prepared["squares"].ptr,
                     float(x.norm[2]), x.rows, out.ptr, out.ld, F.GEMV_MODES[mode], b.status, b.stream, need=b.need_for(x.rows))
            return
        if x.norm is None and ahead is not None and ahead[0] == "rms" and ahead[3] == N and N % 8 == 0 and out.ld == N and self._gemv_fits(N):
            # The RMS norm that reads the stream next: its input times its weight as bfloat16 and the sums of
            # squares come out of this product's epilogue, which has the stream's new values in hand.
            _, weight, eps, _ = ahead
            side = b.temp(x.rows, N, torch.bfloat16)
            squares = b.temp((N + 15) // 16, 8, torch.float32)
            b.launch("gemv_bf16", "mlr_gemv_bf16_add_prepare", w.data_ptr(), w.stride(0), N, K, x.ptr, x.ld, x.rows, out.ptr, out.ld,
                     side.ptr, weight.data_ptr(), native.is_bf16(weight), squares.ptr, b.status, b.stream, need=b.need_for(x.rows))
            b.prepared = {"stream": out.ptr, "weight": weight, "side": side, "squares": squares}
            return
        if x.norm is not None:
            h, weight, eps, wanted_only, _ = x.norm
            source = (h.ptr, h.ld, 1, weight.data_ptr(), native.is_bf16(weight), float(eps), b.meta("want_rows") if wanted_only else None)
        else:
            source = (x.ptr, x.ld, 0, None, 0, 0.0, None)
        b.launch("gemv_bf16", "mlr_gemv_bf16", w.data_ptr(), w.stride(0), N, K, *source, x.rows, out.ptr, out.ld,
                 F.GEMV_MODES[mode], b.status, b.stream, need=b.need_for(x.rows))

    def materialize(self, b, x: Buf) -> Buf:
        """The result of a norm that waited for a product (`Buf.norm`), for a reader that cannot norm its own input."""
        if x.norm is None:
            return x
        h, weight, eps, wanted_only, _ = x.norm
        out = b.temp(x.rows, x.width, x.dtype)
        b.launch("elementwise", "mlr_rmsnorm", h.ptr, None, 1, 0, weight.data_ptr(), native.is_bf16(weight), out.ptr, out.is_bf16,
                 b.meta("want_rows") if wanted_only else None, x.rows, x.width, float(eps), 0, b.stream,
                 need="want" if wanted_only else None)
        x.ptr, x.tensor, x.ld, x.norm = out.ptr, out.tensor, out.ld, None        # every later reader finds the result
        return x

    def linear(self, b, x: Buf, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None, activation: bool = False,
               out: Optional[Buf] = None) -> Buf:
        """x W^T.  `activation`: the result feeds a row-wise kernel as an activation (q/k/v,
        gate/up) rather than the residual stream or the logits."""
        out_dtype = out_dtype or self.dtype
        N, K = w.shape
        if out is None:
            out = b.temp(x.rows, N, torch.float32 if self.dtype is torch.float32 else out_dtype)
        if self._gemv(b, x, w):
            self._gemv_launch(b, x, w, out, "bf16" if out.dtype is torch.bfloat16 else "f32")
            return out
        x = self.materialize(b, x)
        if self.dtype is torch.float32:
            b.launch("gemm_f32", "mlr_gemm_f32", x.ptr, w.data_ptr(), out.ptr, x.rows, N, K, x.ld, w.stride(0), out.ld, b.stream,
                     need=b.need_for(x.rows))
        elif self._pair(b, x, w):
            self._pair_launch(b, x, w, out, "bf16" if out.dtype is torch.bfloat16 else "f32")
        elif (not activation or self.own_activation_products or self.tcgen05_prefill) and self._own_gemm(b, x, w):
            self._own_launch(b, x, w, out)
        else:
            self._library_launch(b, x, w, out)
        return out

    def linear_partials(self, b, x: Buf, w: torch.Tensor, activation: bool = False) -> Optional[Buf]:
        """For the few rows of a decode step: the product as float32 partial sums [S, M, N]
        over S ranges of K (so that a small weight matrix still occupies every SM); the
        kernel that reads them adds them up.  None when the product is not of that kind."""
        if self.dtype is not torch.bfloat16 or (activation and not self.own_activation_products) or self._gemv(b, x, w):
            return None
        x = self.materialize(b, x)
        if not self._tcgen05_ok(x, w) or not b.le(x.rows, self.decode_rows):
            return None
        key = (w.shape[0], w.shape[1])
        splits = self._splits.get(key)
        if splits is None:
            splits = self._splits[key] = executor.k_splits_for(w.shape[0], w.shape[1], self.sm_count)
        out = b.temp(x.rows, w.shape[0], torch.float32, slices=splits)
        self._own_launch(b, x, w, out)
        return out

    def linear_delta(self, b, x: Buf, w: torch.Tensor, into: Optional[Buf] = None) -> Optional[Buf]:
        """A float32 contribution to the residual stream: [M, N], or [S, M, N] partial sums
        that the next norm adds up.  With `into` (the stream itself, float32 [M, N]) the
        product of a prompt portion adds its result there in its epilogue (into += x W^T,
        one rounding per element as the separate add had) and None is returned."""
        direct = into is not None and self.dtype is torch.bfloat16 and into.dtype is torch.float32 and into.ld == into.width
        if direct and self._gemv(b, x, w, adds=True):
            self._gemv_launch(b, x, w, into, "add_f32")
            return None
        parts = self.linear_partials(b, x, w)
        if parts is not None:
            return parts
        x = self.materialize(b, x)
        if direct:
            if self._pair(b, x, w):
                self._pair_launch(b, x, w, into, "add_f32")
                return None
            if not self._own_gemm(b, x, w):
                self._library_launch(b, x, w, into, accumulate=True)
                return None
        return self.linear(b, x, w, out_dtype=torch.float32)

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

    def gated_linear(self, b, x: Buf, w_gate_up: torch.Tensor) -> Buf:
        """silu(x Wgate^T) * (x Wup^T) for the operand `stack_gate_up` made."""
        inter = w_gate_up.shape[0] // 2
        block = F.GATE_BLOCK if self.dtype is torch.bfloat16 else inter
        out = b.temp(x.rows, inter, self.dtype)
        if self._gemv(b, x, w_gate_up) and w_gate_up.shape[0] % (2 * F.GATE_BLOCK) == 0:
            self._gemv_launch(b, x, w_gate_up, out, "silu_gate")
            return out
        x = self.materialize(b, x)
        if self.dtype is torch.bfloat16 and self._pair(b, x, w_gate_up, gated=True):
            self._pair_launch(b, x, w_gate_up, out, "silu_gate")
            return out
        parts = self.linear_partials(b, x, w_gate_up, activation=True)
        if parts is not None:
            b.launch("elementwise", "mlr_swiglu_sliced", parts.ptr, parts.slices, parts.slice_stride, out.ptr, out.is_bf16, x.rows,
                     inter, block, b.stream)
        else:
            both = self.linear(b, x, w_gate_up, activation=True)
            b.launch("elementwise", "mlr_swiglu", both.ptr, out.ptr, out.is_bf16, x.rows, inter, block, b.stream)
        return out
