"""Grouped-query causal attention with per-head q/k RMS norm and rotation, over the
paged cache (src/minillm/runtime.cpp:250-319; src/minillm/cuda/layer.cpp:43-63).

    qkv = x [Wq; Wk; Wv]^T                       one product on the stacked matrices
    q_h, k_h <- rmsnorm over D, then rotate      (skipped when the spec names no norm / position)
    cache[page(pos)] <- k, v                     unless this run reads another run's cache
    o_h = softmax(q_h K^T * scale) V             keys [lo, pos], lo = 0 or pos - window + 1
    delta = o Wo^T                               float32, added to the stream by the next norm

Parameters: hidden_size, num_heads, num_kv_heads, head_dim, scale, window (None or
n), qk_norm_eps (None = no q/k norm), position (name of a position encoding of the
plan, or None).  Weights: "q" [Hq D, H], "k", "v" [Hkv D, H], "o" [H, Hq D],
"q_norm", "k_norm" [D].
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.base import ConfigError
from ..config.registry import register_part
from ..ops import functions as F
from ..ops import attention as A
from ..ops import native
from ..weights.loader import WeightSpec
from .base import CacheNeed, Mixer, RunContext, StepContext


MAX_HEAD_DIM = 256        # the generic kernel keeps two values of a head per thread of its 128


class AttentionMixer(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        p = spec.params
        self.width = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.kv_heads = int(p["num_kv_heads"])
        self.head_dim = int(p["head_dim"])
        self.scale = float(p["scale"])
        self.window = p.get("window")
        self.qk_norm_eps = p.get("qk_norm_eps")
        self.position_name = p.get("position")
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} query heads cannot share {self.kv_heads} kv heads")
        # What no attention kernel of the package takes is refused here, when the plan is built, not at the first step.
        if not 1 <= self.head_dim <= MAX_HEAD_DIM:
            raise ConfigError(f"head size {self.head_dim} is outside what the attention kernels take (1 to {MAX_HEAD_DIM})")
        self.position = None       # set by the model from the plan's position encodings
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = None

    def cache_need(self) -> CacheNeed:
        return CacheNeed(self.window, self.kv_heads, self.head_dim)

    def weight_specs(self) -> List[WeightSpec]:
        w, D = self.spec.weights, self.head_dim
        specs = [WeightSpec(w["q"], (self.heads * D, self.width)), WeightSpec(w["k"], (self.kv_heads * D, self.width)),
                 WeightSpec(w["v"], (self.kv_heads * D, self.width)), WeightSpec(w["o"], (self.width, self.heads * D))]
        if self.qk_norm_eps is not None:
            specs += [WeightSpec(w["q_norm"], (D,), "vector", ("one_plus_normal", 0.01)),
                      WeightSpec(w["k_norm"], (D,), "vector", ("one_plus_normal", 0.01))]
        return specs

    def kernel_modules(self, dtype) -> List[str]:
        return ["elementwise"] + A.modules_for(dtype, self.head_dim) + F.product_modules(dtype)

    def bind(self, tensors: Dict[str, torch.Tensor], rt) -> None:
        w = self.spec.weights
        self.w_qkv = torch.cat([rt.matrix(tensors[w[r]]) for r in ("q", "k", "v")], dim=0).contiguous()
        self.w_o = rt.matrix(tensors[w["o"]])
        if self.qk_norm_eps is not None:
            self.q_norm = rt.vector(tensors[w["q_norm"]])
            self.k_norm = rt.vector(tensors[w["k_norm"]])
            if self.q_norm.dtype is not self.k_norm.dtype:
                self.q_norm, self.k_norm = self.q_norm.float(), self.k_norm.float()

    def emit(self, b, x, run: RunContext):
        rt = b.rt
        D = self.head_dim
        width = self.w_qkv.shape[0]
        partials = rt.linear_partials(b, x, self.w_qkv, activation=True)
        qkv = b.temp(x.rows, width, rt.dtype) if partials is not None else rt.linear(b, x, self.w_qkv, activation=True)
        rotation = self.position.rotation_table() if self.position is not None else None
        if run.write_cache and run.cache.dtype is not qkv.dtype:
            raise native.KernelError(f"cache dtype {run.cache.dtype} differs from activation dtype {qkv.dtype}")
        out = b.temp(x.rows, self.heads * D, rt.dtype)
        # When every segment of a step is a decoded token (or a portion of two or three), the split-KV kernel
        # norms and rotates its own queries and makes the step's keys and values itself: the row-wise kernel
        # below then runs only in steps that also have prompt tiles.
        plan, _ = A.plan_for(b, qkv, out, self.heads, self.kv_heads, D, self.window or 0)
        fused = (plan is not None and partials is None and run.write_cache and (rotation is None or rotation.shape[1] == D)
                 and D <= 256 and rt.fuse_rotation_rows > 0 and b.le(x.rows, rt.fuse_rotation_rows))
        # In place on qkv: per-head RMS norm of q and k, rotation by the table row of each position, and
        # the write of k and v into the run's cache (from the product's partial sums when it left those).
        b.launch("elementwise", "mlr_qk_norm_rope_cache", qkv.ptr, qkv.is_bf16, qkv.ld,
                 partials.ptr if partials is not None else None, partials.slices if partials is not None else 0,
                 partials.slice_stride if partials is not None else 0, partials.ld if partials is not None else 0,
                 x.rows, self.heads, self.kv_heads, D,
                 self.q_norm.data_ptr() if self.q_norm is not None else None,
                 self.k_norm.data_ptr() if self.k_norm is not None else None,
                 native.is_bf16(self.q_norm) if self.q_norm is not None else 0,
                 float(self.qk_norm_eps) if self.qk_norm_eps is not None else 1.0,
                 rotation.data_ptr() if rotation is not None else None,
                 rotation.shape[1] if rotation is not None else 0, rotation.shape[0] if rotation is not None else 0,
                 b.meta("positions"), b.meta("segment_of_row"), b.table(run.group), b.table_stride(run.group), b.page_size,
                 run.cache.data_ptr(), run.cache.shape[0], int(run.write_cache), b.status, b.stream,
                 need=plan.n_prompt_tiles if fused else None)
        fresh = (self.q_norm, self.k_norm, self.qk_norm_eps, rotation) if fused else None
        A.paged_attention(b, qkv, out, run.cache, run.group, self.heads, self.kv_heads, D, self.window or 0, self.scale, fresh=fresh)
        return rt.linear_delta(b, out, self.w_o, into=b.residual)


register_part("mixer", "attention", AttentionMixer)
