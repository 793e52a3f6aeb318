"""Chooses the attention kernel for a step.

float32: the generic kernel (any head size up to 256).  bfloat16: the tensor-core
kernels when they cover the head size, else the generic kernel in bfloat16.
"""
from __future__ import annotations

from typing import List

import torch

from . import functions as F


def modules_for(dtype: torch.dtype, head_dim: int) -> List[str]:
    return ["attention_generic"]


def paged_attention(qkv, out, cache, table, step, q_heads, kv_heads, head_dim, window, scale, cache_group=None):
    """qkv: [M, (Hq + 2 Hkv) D] after norm and rotation (queries in the first Hq D
    columns); out: [M, Hq D]."""
    F.attention_generic(qkv, out, cache, step.positions, step.segment_of_row, table, step.page_size,
                        q_heads, kv_heads, head_dim, window, scale, step.status)
