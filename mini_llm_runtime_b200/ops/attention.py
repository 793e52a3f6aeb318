"""Chooses the attention kernels for a step and plans their launches.

float32: the generic kernel (one block per row and head; any head size up to 256).
bfloat16, head size a multiple of 16: the tensor-core kernels.  Segments that bring
at most 16 rows per kv head (a decoded token, a portion of two or three tokens) go
to the split-KV kernel; the rest are prompt portions and go to the flash kernels: with
head size 64 or 128 (and a page size the kernel takes) in 128-row tiles to the tcgen05
kernel, a remainder of up to 64 rows and everything else in 64-row tiles to the mma.sync
kernel.  A mixed step launches all of them.  Other head sizes in bfloat16 use the generic
kernel.

The plan (which segments go where, how the keys are split) depends only on the
step's segments and on the head grouping, so it is made once per step and reused by
every layer; it is made by the native executor (`plan_attention` in csrc/host/executor.cpp).
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import native


def tensor_core_ok(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def modules_for(dtype: torch.dtype, head_dim: int) -> List[str]:
    if dtype is torch.bfloat16 and tensor_core_ok(head_dim):
        return ["attention_bf16", "attention_tcgen05"] if head_dim in (64, 128) else ["attention_bf16"]
    return ["attention_generic"]


def plan_for(b, qkv, out, q_heads, kv_heads, head_dim, window):
    """The step's launch plan for the bfloat16 tensor-core kernels and whether 128-row tiles may be used, or
    (None, False) when the generic kernel takes the step (float32, other head sizes)."""
    if qkv.dtype is not torch.bfloat16 or not tensor_core_ok(head_dim):
        return None, False
    wide = (getattr(b.rt, "tcgen05_attention", True) and head_dim in (64, 128) and 8 <= b.page_size <= 256
            and b.page_size & (b.page_size - 1) == 0 and qkv.ld % 8 == 0 and out.ld % 8 == 0 and qkv.ptr % 16 == 0
            and out.ptr % 16 == 0)
    return b.plan((q_heads // kv_heads, kv_heads, int(window), int(wide), head_dim, 1)), wide


def paged_attention(b, qkv, out, cache, group, q_heads, kv_heads, head_dim, window, scale, fresh=None):
    """Described to the builder `b` (engine/builder.py): attention of every row of qkv [M, (Hq + 2 Hkv) D]
    (after norm and rotation; queries in the first Hq D columns) over its request's cache, into out
    [M, Hq D].  Which of the bfloat16 kernels run, over which segments and with how many key splits, is
    the step's launch plan (`b.plan`: made by the native executor from the step's segments; it depends
    only on them and on the head grouping, so every layer of a step shares it).

    `fresh` = (q norm weight, k norm weight, eps, rotation table), each possibly None: when every segment of a
    step goes to the split-KV kernel, the row-wise kernel before attention was NOT launched (the caller gave
    it `need=plan.n_prompt_tiles`), qkv is the raw output of the product, and the split-KV kernel norms,
    rotates and writes the cache itself."""
    table, stride = b.table(group), b.table_stride(group)
    plan, wide = plan_for(b, qkv, out, q_heads, kv_heads, head_dim, window)
    if plan is None:
        if cache.dtype is not qkv.dtype or not cache.is_contiguous():
            raise native.KernelError("attention: q, out and cache must share one dtype, and the cache must be contiguous")
        b.launch("attention_generic", "mlr_attention_generic", qkv.ptr, qkv.ld, out.ptr, out.ld, qkv.is_bf16, cache.data_ptr(),
                 cache.shape[0], b.meta("positions"), b.meta("segment_of_row"), table, stride, b.page_size, qkv.rows, q_heads,
                 kv_heads, head_dim, int(window), float(scale), b.status, b.stream)
        return
    if cache.dtype is not torch.bfloat16 or not cache.is_contiguous():
        raise native.KernelError("attention: the bfloat16 kernels take a contiguous bfloat16 cache")
    info = b.meta("segment_info")
    # Segments of few rows (a decoded token, a portion of two or three): split-KV, merged by the last block.
    if fresh is not None:
        q_weight, k_weight, eps, rotation = fresh
        b.launch("attention_bf16", "mlr_attention_decode_fresh_bf16", qkv.ptr, qkv.ld, out.ptr, out.ld, cache.data_ptr(),
                 cache.shape[0], plan.items, plan.n_items, info, table, stride, b.page_size, q_heads, kv_heads, head_dim,
                 int(window), float(scale), plan.chunk, plan.max_splits, plan.scratch, plan.counters,
                 q_weight.data_ptr() if q_weight is not None else None, k_weight.data_ptr() if k_weight is not None else None,
                 native.is_bf16(q_weight) if q_weight is not None else 0, float(eps) if eps is not None else 1.0,
                 rotation.data_ptr() if rotation is not None else None, rotation.shape[0] if rotation is not None else 0,
                 b.status, b.stream, need=plan.n_items_alone)
    b.launch("attention_bf16", "mlr_attention_decode_bf16", qkv.ptr, qkv.ld, out.ptr, out.ld, cache.data_ptr(), cache.shape[0],
             plan.items, plan.n_items, info, table, stride, b.page_size, q_heads, kv_heads, head_dim, int(window), float(scale),
             plan.chunk, plan.max_splits, plan.scratch, plan.counters, b.status, b.stream,
             need=plan.n_items if fresh is None else plan.n_items_beside)
    # Prompt portions: 128-row tiles on the tcgen05 kernel, the rest in 64-row tiles on the mma.sync kernel.
    if wide:
        b.launch("attention_tcgen05", "mlr_attention_prefill_tcgen05", qkv.ptr, qkv.ld, qkv.rows, out.ptr, out.ld,
                 cache.data_ptr(), cache.shape[0], plan.wide_tiles, plan.n_wide, info, table, stride, b.page_size, q_heads,
                 kv_heads, head_dim, int(window), float(scale), b.status, b.stream, need=plan.n_wide)
    b.launch("attention_bf16", "mlr_attention_prefill_bf16", qkv.ptr, qkv.ld, out.ptr, out.ld, cache.data_ptr(), cache.shape[0],
             plan.tiles, plan.n_tiles, info, table, stride, b.page_size, q_heads, kv_heads, head_dim, int(window), float(scale),
             b.status, b.stream, need=plan.n_tiles)
