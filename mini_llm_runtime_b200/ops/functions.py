"""The operations the parts are made of, each one a hand-written kernel launch.

Shapes use M = rows of the step, H = model width.  The residual stream `h` is
always float32; activations are float32 or bfloat16.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .native import call, expect, is_bf16, on_gpu, ptr, stream, KernelError


def embed_gather(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, status: torch.Tensor) -> None:
    """out[r, :] = table[ids[r], :] as float32; an id outside the table zeroes the row
    and sets a status bit."""
    on_gpu(table, ids, out, status)
    expect(ids, torch.int32, "token ids")
    expect(out, torch.float32, "the residual stream")
    rows, width = out.shape
    call("elementwise", "mlr_embed_gather", ptr(out), ptr(table), is_bf16(table), ptr(ids), rows, width,
         table.shape[0], ptr(status), stream())


def rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            delta: Optional[torch.Tensor] = None, rows: Optional[torch.Tensor] = None,
            write_back: bool = True) -> None:
    """out[r] = rmsnorm(h[row] + delta[row]) * weight with row = rows[r] (or r).  With
    `write_back` the sum is stored to h[row], which moves the residual stream on.
    `delta` may be [S, M, H]: S partial sums that are added in order first."""
    on_gpu(h, weight, out, delta, rows)
    expect(h, torch.float32, "the residual stream")
    slices, slice_stride = 1, 0
    if delta is not None:
        expect(delta, torch.float32, "the residual delta")
        if delta.dim() == 3:
            slices, slice_stride = delta.shape[0], delta.stride(0)
        if tuple(delta.shape[-2:]) != tuple(h.shape):
            raise KernelError("residual delta and residual stream differ in shape")
    if rows is not None:
        expect(rows, torch.int32, "row indices")
    count = out.shape[0]
    call("elementwise", "mlr_rmsnorm", ptr(h), ptr(delta), slices, slice_stride, ptr(weight), is_bf16(weight), ptr(out), is_bf16(out),
         ptr(rows), count, h.shape[1], float(eps), int(write_back), stream())


def qk_norm_rope_cache(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int,
                       q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor], eps: float,
                       cos_sin: Optional[torch.Tensor], positions: torch.Tensor, segment_of_row: torch.Tensor,
                       block_table: Optional[torch.Tensor], page_size: int, cache: Optional[torch.Tensor],
                       write_cache: bool, status: torch.Tensor, partials: Optional[torch.Tensor] = None) -> None:
    """In place on qkv [M, (Hq + 2 Hkv) D]: per-head RMS norm of q and k, rotation by
    the table row of each position, and the write of k and v into the layer's cache
    [page, 2, Hkv, page_size, D].  With `partials` (float32 [S, M, width]) the input is the
    sum of those slices instead, and qkv only receives the results."""
    on_gpu(qkv, q_weight, k_weight, cos_sin, positions, segment_of_row, block_table, cache, status, partials)
    slices, slice_stride, ld_partial = 0, 0, 0
    if partials is not None:
        expect(partials, torch.float32, "the partial sums")
        if partials.dim() != 3 or partials.shape[1] != qkv.shape[0]:
            raise KernelError("qk_norm_rope_cache: partial sums must be [S, M, width]")
        slices, slice_stride, ld_partial = partials.shape[0], partials.stride(0), partials.stride(1)
    expect(positions, torch.int32, "positions")
    expect(segment_of_row, torch.int32, "segment_of_row")
    if cos_sin is not None:
        expect(cos_sin, torch.float32, "the rotation table")
    if write_cache:
        expect(block_table, torch.int32, "the block table")
        if cache.dtype is not qkv.dtype:
            raise KernelError(f"cache dtype {cache.dtype} differs from activation dtype {qkv.dtype}")
    w_bf16 = is_bf16(q_weight) if q_weight is not None else 0
    call("elementwise", "mlr_qk_norm_rope_cache", ptr(qkv), is_bf16(qkv), qkv.stride(0), ptr(partials), slices,
         slice_stride, ld_partial, qkv.shape[0], q_heads,
         kv_heads, head_dim, ptr(q_weight), ptr(k_weight), w_bf16, float(eps), ptr(cos_sin),
         cos_sin.shape[1] if cos_sin is not None else 0, cos_sin.shape[0] if cos_sin is not None else 0,
         ptr(positions), ptr(segment_of_row), ptr(block_table),
         block_table.stride(0) if block_table is not None else 0, page_size, ptr(cache),
         cache.shape[0] if cache is not None else 0, int(write_cache), ptr(status), stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0) -> None:
    """out[M, I] = silu(gate) * up for gate_up [M, 2 I] laid out in blocks of `block` gate
    columns followed by the `block` "up" columns of the same outputs; block = 0 means I
    (all gates, then all ups).  gate_up may also be float32 [S, M, 2 I]: S partial sums
    that are added in order first."""
    on_gpu(gate_up, out)
    block = block or out.shape[1]
    if out.shape[1] % block:
        raise KernelError(f"swiglu: the width {out.shape[1]} is no multiple of the gate block {block}")
    if gate_up.dim() == 3:
        expect(gate_up, torch.float32, "the partial sums")
        if not out.is_contiguous() or gate_up.shape[2] != 2 * out.shape[1] or gate_up.shape[1] != out.shape[0]:
            raise KernelError("swiglu: partial sums [S, M, 2 I] do not fit the output [M, I]")
        call("elementwise", "mlr_swiglu_sliced", ptr(gate_up), gate_up.shape[0], gate_up.stride(0), ptr(out), is_bf16(out),
             out.shape[0], out.shape[1], block, stream())
        return
    if not gate_up.is_contiguous() or not out.is_contiguous() or gate_up.dtype is not out.dtype:
        raise KernelError("swiglu wants contiguous tensors of one dtype")
    if gate_up.shape != (out.shape[0], 2 * out.shape[1]):
        raise KernelError(f"swiglu: gate_up {tuple(gate_up.shape)} does not fit the output {tuple(out.shape)}")
    call("elementwise", "mlr_swiglu", ptr(gate_up), ptr(out), is_bf16(out), out.shape[0], out.shape[1], block, stream())


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 on the CUDA cores."""
    on_gpu(a, w, out)
    for t, what in ((a, "a"), (w, "w"), (out, "out")):
        if t.dtype is not torch.float32 or t.stride(1) != 1:
            raise KernelError(f"gemm_f32: {what} must be float32 with unit inner stride")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N):
        raise KernelError(f"gemm_f32: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not fit")
    call("gemm_f32", "mlr_gemm_f32", ptr(a), ptr(w), ptr(out), M, N, K, a.stride(0), w.stride(0), out.stride(0), stream())


def attention_generic(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                      segment_of_row: torch.Tensor, block_table: torch.Tensor, page_size: int, q_heads: int,
                      kv_heads: int, head_dim: int, window: int, scale: float, status: torch.Tensor) -> None:
    """Causal (optionally windowed) attention of every row over its request's cache.
    q is [M, >= Hq*D] (a view into the qkv buffer is fine), out is [M, Hq*D]."""
    on_gpu(q, out, cache, positions, segment_of_row, block_table, status)
    if q.dtype is not out.dtype or q.dtype is not cache.dtype:
        raise KernelError("attention: q, out and cache must share one dtype")
    if q.stride(1) != 1 or out.stride(1) != 1 or not cache.is_contiguous():
        raise KernelError("attention: inner strides must be 1 and the cache contiguous")
    call("attention_generic", "mlr_attention_generic", ptr(q), q.stride(0), ptr(out), out.stride(0), is_bf16(q),
         ptr(cache), cache.shape[0], ptr(positions), ptr(segment_of_row), ptr(block_table), block_table.stride(0),
         page_size, q.shape[0], q_heads, kv_heads, head_dim, int(window), float(scale), ptr(status), stream())


def sample(logits: torch.Tensor, out: torch.Tensor, status: torch.Tensor,
           temperature: Optional[torch.Tensor] = None, uniform: Optional[torch.Tensor] = None) -> None:
    """out[r] = greedy choice of logits[r] (temperature 0) or an inverse-CDF draw with
    the row's uniform number."""
    on_gpu(logits, out, status, temperature, uniform)
    expect(out, torch.int32, "sampled ids")
    if logits.dtype is not torch.float32 or logits.stride(1) != 1:
        raise KernelError("sample: logits must be float32 rows")
    if temperature is not None:
        expect(temperature, torch.float32, "temperatures")
        expect(uniform, torch.float64, "uniform numbers")
    call("sampling", "mlr_sample", ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1],
         ptr(temperature), ptr(uniform), ptr(out), ptr(status), stream())


def attention_decode_bf16(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, items: Optional[torch.Tensor],
                          n_items: int, segment_info: torch.Tensor, block_table: torch.Tensor, page_size: int,
                          q_heads: int, kv_heads: int, head_dim: int, window: int, scale: float, chunk: int,
                          max_splits: int, partial: Optional[torch.Tensor], status: torch.Tensor,
                          counters: Optional[torch.Tensor] = None) -> None:
    """Split-KV attention for requests that bring at most 16 rows per kv head (tokens
    times query heads per kv head).  `items` lists the segments to run (None: all of
    them, in order); `partial` is float32 scratch of `attention_decode_scratch_floats`
    elements and `counters` int32 zeros, one per item and kv head, which the kernel leaves
    zero again (both needed when max_splits > 1; without `counters` a zeroed tensor is made)."""
    on_gpu(q, out, cache, items, segment_info, block_table, partial, status, counters)
    if max_splits > 1 and counters is None:
        counters = torch.zeros(n_items * kv_heads, dtype=torch.int32, device=q.device)
    if counters is not None:
        expect(counters, torch.int32, "the split counters")
        if counters.numel() < n_items * kv_heads:
            raise KernelError("attention_decode_bf16: too few split counters")
    for t in (q, out, cache):
        if t.dtype is not torch.bfloat16:
            raise KernelError("attention_decode_bf16 takes bfloat16 tensors")
    if q.stride(1) != 1 or out.stride(1) != 1 or not cache.is_contiguous():
        raise KernelError("attention: inner strides must be 1 and the cache contiguous")
    if partial is not None:
        expect(partial, torch.float32, "the split scratch")
        if partial.numel() < attention_decode_scratch_floats(n_items, kv_heads, head_dim, max_splits):
            raise KernelError("attention_decode_bf16: the split scratch is too small")
    call("attention_bf16", "mlr_attention_decode_bf16", ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache),
         cache.shape[0], ptr(items), n_items, ptr(segment_info), ptr(block_table), block_table.stride(0), page_size,
         q_heads, kv_heads, head_dim, int(window), float(scale), int(chunk), int(max_splits), ptr(partial),
         ptr(counters), ptr(status), stream())


def attention_decode_fresh_bf16(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, items: Optional[torch.Tensor],
                                n_items: int, segment_info: torch.Tensor, block_table: torch.Tensor, page_size: int,
                                q_heads: int, kv_heads: int, head_dim: int, window: int, scale: float, chunk: int,
                                max_splits: int, partial: Optional[torch.Tensor], q_weight: Optional[torch.Tensor],
                                k_weight: Optional[torch.Tensor], eps: float, cos_sin: Optional[torch.Tensor],
                                status: torch.Tensor, counters: Optional[torch.Tensor] = None) -> None:
    """`attention_decode_bf16` over the RAW output of the q/k/v product [M, (Hq + 2 Hkv) D]: the kernel norms q and k
    per head, rotates them by the table row of each token's position, writes the step's k and v into the cache and
    attends; it stands for `qk_norm_rope_cache` followed by `attention_decode_bf16` when every segment of the step is
    one of `items`.  qkv is left as it was."""
    on_gpu(qkv, out, cache, items, segment_info, block_table, partial, status, counters, q_weight, k_weight, cos_sin)
    if max_splits > 1 and counters is None:
        counters = torch.zeros(n_items * kv_heads, dtype=torch.int32, device=qkv.device)
    for t in (qkv, out, cache):
        if t.dtype is not torch.bfloat16:
            raise KernelError("attention_decode_fresh_bf16 takes bfloat16 tensors")
    if qkv.stride(1) != 1 or out.stride(1) != 1 or not cache.is_contiguous():
        raise KernelError("attention: inner strides must be 1 and the cache contiguous")
    if cos_sin is not None:
        expect(cos_sin, torch.float32, "the rotation table")
        if cos_sin.shape[1] != head_dim or not cos_sin.is_contiguous():
            raise KernelError("attention_decode_fresh_bf16: the rotation table must be [positions, head_dim]")
    if q_weight is not None and k_weight is not None and q_weight.dtype is not k_weight.dtype:
        raise KernelError("attention_decode_fresh_bf16: q and k norm weights must share a dtype")
    if partial is not None:
        expect(partial, torch.float32, "the split scratch")
        if partial.numel() < attention_decode_scratch_floats(n_items, kv_heads, head_dim, max_splits):
            raise KernelError("attention_decode_fresh_bf16: the split scratch is too small")
    call("attention_bf16", "mlr_attention_decode_fresh_bf16", ptr(qkv), qkv.stride(0), ptr(out), out.stride(0), ptr(cache),
         cache.shape[0], ptr(items), n_items, ptr(segment_info), ptr(block_table), block_table.stride(0), page_size,
         q_heads, kv_heads, head_dim, int(window), float(scale), int(chunk), int(max_splits), ptr(partial), ptr(counters),
         ptr(q_weight), ptr(k_weight), is_bf16(q_weight) if q_weight is not None else 0, float(eps), ptr(cos_sin),
         cos_sin.shape[0] if cos_sin is not None else 0, ptr(status), stream())


def attention_decode_scratch_floats(n_items: int, kv_heads: int, head_dim: int, max_splits: int) -> int:
    return n_items * kv_heads * max_splits * 16 * (head_dim + 2)


def attention_prefill_bf16(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor,
                           segment_info: torch.Tensor, block_table: torch.Tensor, page_size: int, q_heads: int,
                           kv_heads: int, head_dim: int, window: int, scale: float, status: torch.Tensor) -> None:
    """Flash attention for prompt portions.  `tiles` is int32 [n, 2]: segment index and
    first token of each 64-row tile."""
    on_gpu(q, out, cache, tiles, segment_info, block_table, status)
    for t in (q, out, cache):
        if t.dtype is not torch.bfloat16:
            raise KernelError("attention_prefill_bf16 takes bfloat16 tensors")
    if q.stride(1) != 1 or out.stride(1) != 1 or not cache.is_contiguous():
        raise KernelError("attention: inner strides must be 1 and the cache contiguous")
    expect(tiles, torch.int32, "the tile list")
    call("attention_bf16", "mlr_attention_prefill_bf16", ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(cache),
         cache.shape[0], ptr(tiles), tiles.shape[0], ptr(segment_info), ptr(block_table), block_table.stride(0),
         page_size, q_heads, kv_heads, head_dim, int(window), float(scale), ptr(status), stream())


def attention_prefill_tcgen05_applies(q: torch.Tensor, out: torch.Tensor, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 prompt-attention kernel takes these tensors (head size 64 or 128,
    a page size that is a power of two from 8 to 256, 16-byte aligned rows)."""
    return (head_dim in (64, 128) and 8 <= page_size <= 256 and page_size & (page_size - 1) == 0
            and q.dtype is torch.bfloat16 and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0
            and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0)


def attention_prefill_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, tiles: torch.Tensor,
                              segment_info: torch.Tensor, block_table: torch.Tensor, page_size: int, q_heads: int,
                              kv_heads: int, head_dim: int, window: int, scale: float, status: torch.Tensor) -> None:
    """Flash attention for prompt portions on the tcgen05 tensor cores.  `tiles` is int32
    [n, 2]: segment index and first token of each 128-row tile."""
    on_gpu(q, out, cache, tiles, segment_info, block_table, status)
    for t in (q, out, cache):
        if t.dtype is not torch.bfloat16:
            raise KernelError("attention_prefill_tcgen05 takes bfloat16 tensors")
    if q.stride(1) != 1 or out.stride(1) != 1 or not cache.is_contiguous():
        raise KernelError("attention: inner strides must be 1 and the cache contiguous")
    expect(tiles, torch.int32, "the tile list")
    call("attention_tcgen05", "mlr_attention_prefill_tcgen05", ptr(q), q.stride(0), q.shape[0], ptr(out), out.stride(0),
         ptr(cache), cache.shape[0], ptr(tiles), tiles.shape[0], ptr(segment_info), ptr(block_table),
         block_table.stride(0), page_size, q_heads, kv_heads, head_dim, int(window), float(scale), ptr(status), stream())


def finite_check(t: torch.Tensor, flag: torch.Tensor) -> None:
    """flag[0] = 1 if `t` (float32 or bfloat16, contiguous) holds a NaN or an infinity."""
    on_gpu(t, flag)
    expect(flag, torch.int32, "the flag")
    if not t.is_contiguous():
        raise KernelError("finite_check wants a contiguous tensor")
    call("weights", "mlr_finite_check", ptr(t), is_bf16(t), t.numel(), ptr(flag), stream())


GEMV_MODES = {"bf16": 0, "f32": 1, "add_f32": 2, "silu_gate": 3}


def _gemv_operands(w: torch.Tensor, x: torch.Tensor, out: torch.Tensor, mode: str, x_dtype: torch.dtype) -> None:
    N, K = w.shape
    if w.dtype is not torch.bfloat16 or w.stride(1) != 1 or x.stride(1) != 1 or out.stride(1) != 1:
        raise KernelError("gemv_bf16: bfloat16 weights and unit inner strides are wanted")
    if x.dtype is not x_dtype or x.shape[1] != K:
        raise KernelError("gemv_bf16: x must be bfloat16 [M, K], or the float32 stream when a norm weight is given")
    columns = N // 2 if mode == "silu_gate" else N
    want = torch.bfloat16 if mode in ("bf16", "silu_gate") else torch.float32
    if out.shape[1] != columns or out.dtype is not want:
        raise KernelError(f"gemv_bf16: an output {tuple(out.shape)} of {out.dtype} does not fit mode {mode!r}")


def gemv_bf16(w: torch.Tensor, x: torch.Tensor, out: torch.Tensor, mode: str = "bf16", norm_weight: Optional[torch.Tensor] = None,
              eps: float = 0.0, rows: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """out = f(x w^T) for one to eight rows (a pass over the weights).  x is bfloat16 [M, K];
    or, with `norm_weight`, the float32 residual stream, of which row r (row rows[r] when `rows` is given)
    is RMS-normed first.  `mode`: "bf16" / "f32" store, "add_f32" adds into the float32 out, "silu_gate"
    takes w as a stacked gate/up matrix (`interleave_gate_up`) and stores silu(gate) * up in out [M, N / 2]."""
    on_gpu(w, x, out, norm_weight, rows, status)
    M = out.shape[0]
    N, K = w.shape
    norm = norm_weight is not None
    _gemv_operands(w, x, out, mode, torch.float32 if norm else torch.bfloat16)
    if not norm and x.shape[0] != M:
        raise KernelError(f"gemv_bf16: {x.shape[0]} rows of x for {M} rows of out")
    if rows is not None:
        expect(rows, torch.int32, "row indices")
    call("gemv_bf16", "mlr_gemv_bf16", ptr(w), w.stride(0), N, K, ptr(x), x.stride(0), int(norm), ptr(norm_weight),
         is_bf16(norm_weight) if norm else 0, float(eps), ptr(rows), M, ptr(out), out.stride(0), GEMV_MODES[mode], ptr(status), stream())


def gemv_bf16_add_prepare(w: torch.Tensor, x: torch.Tensor, out: torch.Tensor, norm_weight: torch.Tensor, side: torch.Tensor,
                          squares: torch.Tensor, status: Optional[torch.Tensor] = None) -> None:
    """out += x w^T as `gemv_bf16` in mode "add_f32", and for the RMS norm with `norm_weight` that reads out next:
    side [M, N] bfloat16 = the new out times the weight, squares [ceil(N / 16), 8] float32 = the sums of squares
    of 16 columns of out per row (`gemv_bf16_prepared` takes both)."""
    on_gpu(w, x, out, norm_weight, side, squares, status)
    M, N = out.shape
    _gemv_operands(w, x, out, "add_f32", torch.bfloat16)
    if (side.dtype is not torch.bfloat16 or tuple(side.shape) != (M, N) or not side.is_contiguous() or squares.dtype is not torch.float32
            or tuple(squares.shape) != ((N + 15) // 16, 8) or not squares.is_contiguous() or norm_weight.shape[0] != N):
        raise KernelError("gemv_bf16_add_prepare: side is bfloat16 [M, N], squares float32 [ceil(N / 16), 8], the weight [N]")
    call("gemv_bf16", "mlr_gemv_bf16_add_prepare", ptr(w), w.stride(0), N, w.shape[1], ptr(x), x.stride(0), M, ptr(out), out.stride(0),
         ptr(side), ptr(norm_weight), is_bf16(norm_weight), ptr(squares), ptr(status), stream())


def gemv_bf16_prepared(w: torch.Tensor, side: torch.Tensor, squares: torch.Tensor, eps: float, out: torch.Tensor, mode: str = "bf16",
                       status: Optional[torch.Tensor] = None) -> None:
    """out = f(n w^T) where n is the RMS norm that `gemv_bf16_add_prepare` left half done in `side` and `squares`."""
    on_gpu(w, side, squares, out, status)
    _gemv_operands(w, side, out, mode, torch.bfloat16)
    if not side.is_contiguous() or tuple(squares.shape) != ((w.shape[1] + 15) // 16, 8) or side.shape[0] != out.shape[0]:
        raise KernelError("gemv_bf16_prepared: side and squares are not what gemv_bf16_add_prepare leaves for this width")
    call("gemv_bf16", "mlr_gemv_bf16_prepared", ptr(w), w.stride(0), w.shape[0], w.shape[1], ptr(side), ptr(squares), float(eps),
         out.shape[0], ptr(out), out.stride(0), GEMV_MODES[mode], ptr(status), stream())


def product_modules(dtype) -> list:
    """The kernel modules the matrix products of a precision may call."""
    return ["gemm_f32"] if dtype is torch.float32 else ["gemv_bf16", "gemm_bf16_tcgen05", "gemm_bf16_tcgen05_pair"]


def gemm_tcgen05_applies(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype is torch.bfloat16 and w.dtype is torch.bfloat16 and x.shape[1] % 8 == 0 and x.shape[1] >= 8
            and x.stride(1) == 1 and w.stride(1) == 1 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_bf16_tcgen05(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor, tile_q: int = 0) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (bf16 in, float32
    accumulate in tensor memory, out bf16 or float32).  With up to 64 rows of x the weight
    matrix takes the 128-row side of the instruction and the result is stored transposed
    (the product is then a single pass over the weights); otherwise x takes that side.

    `out` may also be float32 [S, M, N]: K is then cut into S ranges and slice s holds the
    sum over range s (more thread blocks share a small matrix); the reader adds the slices.

    `w` must hold weights: nothing that runs before this call on the stream may still be
    writing it, because the kernel starts to fetch it before the kernels before it are done."""
    on_gpu(x, w, out, status)
    if not gemm_tcgen05_applies(x, w):
        raise KernelError("gemm_bf16_tcgen05: operands must be bfloat16, K-contiguous, 16-byte aligned, K % 8 == 0")
    if out.dtype not in (torch.bfloat16, torch.float32) or out.stride(-1) != 1:
        raise KernelError("gemm_bf16_tcgen05: the output must be bfloat16 or float32 with unit inner stride")
    M, K = x.shape
    N = w.shape[0]
    splits, split_stride = 1, 0
    if out.dim() == 3:
        splits, split_stride = out.shape[0], out.stride(0)
        if out.dtype is not torch.float32:
            raise KernelError("gemm_bf16_tcgen05: split results must be float32")
    if w.shape[1] != K or tuple(out.shape[-2:]) != (M, N):
        raise KernelError(f"gemm_bf16_tcgen05: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)} do not fit")
    f32 = int(out.dtype is torch.float32)
    ldo = out.stride(-2)
    if M <= 64:
        call("gemm_bf16_tcgen05", "mlr_gemm_bf16_tcgen05", ptr(w), w.stride(0), N, ptr(x), x.stride(0), M, K, ptr(out),
             ldo, f32, 1, tile_q, splits, split_stride, 1, ptr(status), stream())
    else:
        call("gemm_bf16_tcgen05", "mlr_gemm_bf16_tcgen05", ptr(x), x.stride(0), M, ptr(w), w.stride(0), N, K, ptr(out),
             ldo, f32, 0, tile_q, splits, split_stride, 2, ptr(status), stream())


PAIR_EPILOGUES = {"bf16": 0, "f32": 1, "add_f32": 2, "silu_gate": 3}


def gemm_bf16_tcgen05_pair(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, status: torch.Tensor, epilogue: str) -> None:
    """The product x[M, K] @ w[N, K]^T of a prompt portion on pairs of SMs (256 x 256 tiles,
    tcgen05 instructions that span two thread blocks).  `epilogue`: "bf16" or "f32" store the
    result in out[M, N]; "add_f32" adds it to the float32 out[M, N]; "silu_gate" takes w as
    blocks of 128 gate rows, each followed by its 128 "up" rows (`interleave_gate_up`), and
    stores silu(gate) * up in the bfloat16 out[M, N / 2]."""
    on_gpu(x, w, out, status)
    if not gemm_tcgen05_applies(x, w):
        raise KernelError("gemm_bf16_tcgen05_pair: operands must be bfloat16, K-contiguous, 16-byte aligned, K % 8 == 0")
    M, K = x.shape
    N = w.shape[0]
    columns = N // 2 if epilogue == "silu_gate" else N
    want = torch.bfloat16 if epilogue in ("bf16", "silu_gate") else torch.float32
    if w.shape[1] != K or tuple(out.shape) != (M, columns) or out.dtype is not want or out.stride(1) != 1:
        raise KernelError(f"gemm_bf16_tcgen05_pair: {tuple(x.shape)} x {tuple(w.shape)}^T with epilogue {epilogue!r} "
                          f"does not fit an output {tuple(out.shape)} of {out.dtype}")
    call("gemm_bf16_tcgen05_pair", "mlr_gemm_bf16_tcgen05_pair", ptr(x), x.stride(0), M, ptr(w), w.stride(0), N, K, ptr(out),
         out.stride(0), PAIR_EPILOGUES[epilogue], ptr(status), stream())


GATE_BLOCK = 128     # rows of the gate that alternate with their "up" rows in the interleaved operand


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """The stacked matrix the gated epilogue of the pair product reads: 128 rows of the gate,
    then the 128 rows of "up" for the same outputs, and so on; the last block is padded with
    zero rows, so the result has 2 * ceil(I / 128) * 128 rows."""
    inter, K = w_gate.shape
    blocks = -(-inter // GATE_BLOCK)
    padded = torch.zeros((2, blocks * GATE_BLOCK, K), dtype=w_gate.dtype, device=w_gate.device)
    padded[0, :inter] = w_gate
    padded[1, :inter] = w_up
    return padded.view(2, blocks, GATE_BLOCK, K).transpose(0, 1).reshape(2 * blocks * GATE_BLOCK, K)


def k_splits_for(rows: int, K: int, sms: int) -> int:
    """How many ranges to cut K into when a weight matrix of `rows` rows is streamed in tiles
    of 128 rows by `sms` blocks at a time (decided by the native executor, `mlr_k_splits`)."""
    from ..engine.executor import k_splits_for as native_k_splits
    return native_k_splits(rows, K, sms)
