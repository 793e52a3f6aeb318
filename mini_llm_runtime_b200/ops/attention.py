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
every layer.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import functions as F

_TILE = 64
_WIDE_TILE = 128
_MIN_CHUNK = 128


def tensor_core_ok(head_dim: int) -> bool:
    return head_dim % 16 == 0 and 16 <= head_dim <= 256


def modules_for(dtype: torch.dtype, head_dim: int) -> List[str]:
    if dtype is torch.bfloat16 and tensor_core_ok(head_dim):
        return ["attention_bf16", "attention_tcgen05"] if head_dim in (64, 128) else ["attention_bf16"]
    return ["attention_generic"]


def split_plan(spans: List[int], blocks_per_split: int):
    """Keys per split (a multiple of 64) and the largest number of splits, for items
    whose key spans (from a 64-aligned base to the last key) are `spans`.

    `blocks_per_split` thread blocks run for every split (items times kv heads).  Two
    blocks fit an SM.  More splits give smaller blocks (less imbalance, more SMs busy
    when there are few requests) but each block pays a fixed start and merge cost, and a
    last, partly filled wave of blocks costs as much as a full one.  The split count
    with the smallest estimated time wins."""
    longest = max(spans)
    slots = 148 * 2
    per_key_ns, per_block_ns = 0.022, 5.0       # one block streaming beside another; start + merge
    best = None
    limit = max(1, min(512, -(-longest // _MIN_CHUNK)))
    for splits in range(1, limit + 1):
        chunk = -(-(-(-longest // splits)) // _TILE) * _TILE
        real = -(-longest // chunk)
        waves = -(-(real * blocks_per_split) // slots)
        share = min(1.0, real * blocks_per_split / slots / waves * 2)      # SMs with one block stream faster
        estimate = waves * (chunk * per_key_ns * max(share, 0.5) + per_block_ns)
        if best is None or estimate < best[0] - 1e-9:
            best = (estimate, chunk, real)
    return best[1], best[2]


class _Plan:
    pass


def _plan(step, group: int, kv_heads: int, window: int, wide: bool) -> _Plan:
    key = ("attention_plan", group, kv_heads, window, wide)
    plan = step.scratch.get(key)
    if plan is not None:
        return plan
    plan = _Plan()
    device = step.positions.device
    small = [i for i, s in enumerate(step.segments) if group <= 16 and s.count * group <= 16]
    large = [i for i in range(len(step.segments)) if i not in set(small)] if len(small) < len(step.segments) else []
    plan.n_items = len(small)
    plan.items = None
    plan.tiles = None
    plan.wide_tiles = None
    if small:
        if len(small) != len(step.segments):
            plan.items = torch.tensor(small, dtype=torch.int32).to(device)
        spans = []
        for i in small:
            s = step.segments[i]
            if step.context_bound is None:
                first = max(0, s.start - window + 1) if window else 0
                spans.append(s.start + s.count - (first // _TILE) * _TILE)
            else:       # a captured step: plan for the longest context the graph may be replayed with
                spans.append(min(step.context_bound, window + s.count + _TILE) if window else step.context_bound)
        plan.chunk, plan.max_splits = split_plan(spans, len(small) * kv_heads)
    if large:
        tiles, wide_tiles = [], []
        for i in large:
            count = step.segments[i].count
            # 128-row tiles while more than 64 rows are left, then one 64-row tile for the rest.
            cut = 0
            while wide and count - cut > _TILE:
                wide_tiles.append((i, cut))
                cut += _WIDE_TILE
            tiles.extend((i, t) for t in range(cut, count, _TILE))
        longest_first = lambda it: -(step.segments[it[0]].start + it[1])      # longest key walks first
        if tiles:
            plan.tiles = torch.tensor(sorted(tiles, key=longest_first), dtype=torch.int32).to(device)
        if wide_tiles:
            plan.wide_tiles = torch.tensor(sorted(wide_tiles, key=longest_first), dtype=torch.int32).to(device)
    step.scratch[key] = plan
    return plan


def paged_attention(qkv, out, cache, table, step, q_heads, kv_heads, head_dim, window, scale, cache_group=None):
    """qkv: [M, (Hq + 2 Hkv) D] after norm and rotation (queries in the first Hq D
    columns); out: [M, Hq D]."""
    if qkv.dtype is not torch.bfloat16 or not tensor_core_ok(head_dim):
        F.attention_generic(qkv, out, cache, step.positions, step.segment_of_row, table, step.page_size,
                            q_heads, kv_heads, head_dim, window, scale, step.status)
        return
    wide = getattr(step.rt, "tcgen05_attention", True) and F.attention_prefill_tcgen05_applies(qkv, out, head_dim, step.page_size)
    plan = _plan(step, q_heads // kv_heads, kv_heads, window, wide)
    if plan.n_items:
        partial = None
        if plan.max_splits > 1:
            count = F.attention_decode_scratch_floats(plan.n_items, kv_heads, head_dim, plan.max_splits)
            partial = step.scratch.get(("attention_partial", count))
            if partial is None:
                partial = torch.empty(count, dtype=torch.float32, device=qkv.device)
                step.scratch[("attention_partial", count)] = partial
        F.attention_decode_bf16(qkv, out, cache, plan.items, plan.n_items, step.segment_info, table, step.page_size,
                                q_heads, kv_heads, head_dim, window, scale, plan.chunk, plan.max_splits, partial,
                                step.status, counters=step.rt.split_counters(plan.n_items * kv_heads))
    if plan.wide_tiles is not None:
        F.attention_prefill_tcgen05(qkv, out, cache, plan.wide_tiles, step.segment_info, table, step.page_size, q_heads,
                                    kv_heads, head_dim, window, scale, step.status)
    if plan.tiles is not None:
        F.attention_prefill_bf16(qkv, out, cache, plan.tiles, step.segment_info, table, step.page_size, q_heads,
                                 kv_heads, head_dim, window, scale, step.status)
