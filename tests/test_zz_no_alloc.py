"""The decode-attention entry point that allocates no device memory.

Some programs that embed this library cannot call cudaMalloc: all device memory
belongs to their own manager, or they run a loop whose latency an allocator call
would break.  `mlr_attention_decode_bf16_no_alloc` keeps the partial results of the
key splits in an array that is part of the library's device image instead of a
caller's buffer.  This test calls it through its exported C symbol, twice in a row
(the second call finds the first call's leftovers in the array), and wants the same
output as the normal entry point given a scratch buffer, and the same as a plain float64
attention over the same cache.  The driver's count of free device memory must not move
across a call.  A call too large for the array, or with more requests and kv heads than
the built-in counters, is refused.

The file sorts last so that a run that stops at the first failure has run every
other test before it.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_no_alloc_entry_point_matches_the_normal_one():
    from mini_llm_runtime_b200.ops import functions as F
    from mini_llm_runtime_b200.ops import native

    lib = native.module("attention_bf16")
    fn = lib.mlr_attention_decode_bf16_no_alloc
    c_int, c_float, c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
    fn.argtypes = [c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int,
                   c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_void_p, c_void_p]
    fn.restype = c_int

    g = torch.Generator().manual_seed(0)
    Hq, Hkv, D, page = 8, 2, 128, 16
    contexts = [700, 64, 1, 333]
    n = len(contexts)
    blocks = [-(-c // page) for c in contexts]
    pages = sum(blocks)
    cache = (torch.randn(pages, 2, Hkv, page, D, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    for i, b in enumerate(blocks):
        table[i, :b] = torch.tensor([order.pop() for _ in range(b)], dtype=torch.int32)
    table = table.to(DEV)
    info = torch.tensor([[i, 1, c - 1, i] for i, c in enumerate(contexts)], dtype=torch.int32, device=DEV)
    scale, chunk = 1 / math.sqrt(D), 128
    splits = -(-max(contexts) // chunk)
    stream = torch.cuda.current_stream().cuda_stream

    def call_no_alloc(qkv, out, status):
        return fn(qkv.data_ptr(), qkv.stride(0), out.data_ptr(), out.stride(0), cache.data_ptr(), pages, None, n,
                  info.data_ptr(), table.data_ptr(), table.stride(0), page, Hq, Hkv, D, 0, scale, chunk, splits,
                  status.data_ptr(), stream)

    for round_ in range(2):          # two calls in a row share the built-in array
        qkv = torch.randn(n, (Hq + 2 * Hkv) * D, generator=g).to(torch.bfloat16).to(DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        want = torch.full((n, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(F.attention_decode_scratch_floats(n, Hkv, D, splits), device=DEV)
        F.attention_decode_bf16(qkv, want, cache, None, n, info, table, page, Hq, Hkv, D, 0, scale, chunk, splits,
                                partial, status)
        got = torch.full((n, Hq * D), float("nan"), dtype=torch.bfloat16, device=DEV)
        torch.cuda.synchronize()
        # Free memory as the driver counts it: an allocation inside the library would show here
        # (torch's own counters would not see it).  The first call may still load the kernel's
        # module, so the figure is compared across the second call.
        free_before = torch.cuda.mem_get_info()[0]
        assert call_no_alloc(qkv, got, status) == 0, lib.mlr_last_error().decode()
        torch.cuda.synchronize()
        if round_ == 1:
            assert torch.cuda.mem_get_info()[0] == free_before, "device memory was taken during the call"
        assert status.item() == 0 and torch.isfinite(got.float()).all()
        # Same kernels, same order of summation: the tolerance of the kernel tests holds with room to spare.
        assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), f"call {round_}"
        assert torch.equal(got, want), f"call {round_}"
        # A second witness that shares no code with either entry point: dense float64 attention.
        plain = torch.empty(n, Hq, D, dtype=torch.float64)
        host_cache, host_table, q = cache.float().cpu(), table.cpu(), qkv[:, :Hq * D].float().cpu().view(n, Hq, D)
        for i, c in enumerate(contexts):
            position = torch.arange(c)
            rows = host_cache[host_table[i, position // page].long(), :, :, position % page]        # [c, 2, Hkv, D]
            column = torch.arange(D)[None, :] ^ ((position[:, None] & 7) << 3)                       # the cache's stored order
            rows = torch.gather(rows, 3, column[:, None, None, :].expand(c, 2, Hkv, D))
            k, v = (rows[:, j].double().repeat_interleave(Hq // Hkv, 1) for j in (0, 1))             # [c, Hq, D]
            p = torch.softmax(torch.einsum("hd,thd->ht", q[i].double(), k) * scale, dim=-1)
            plain[i] = torch.einsum("ht,thd->hd", p, v)
        assert torch.allclose(got.float().cpu().double().view(n, Hq, D), plain, atol=2e-2, rtol=2e-2), f"call {round_}"

    # A call that needs more scratch than the array holds is refused before any launch.
    too_many = 1 << 20
    code = fn(qkv.data_ptr(), qkv.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), pages, None, n,
              info.data_ptr(), table.data_ptr(), table.stride(0), page, Hq, Hkv, D, 0, scale, 64, too_many,
              status.data_ptr(), stream)
    assert code != 0 and "the built-in array holds" in lib.mlr_last_error().decode()
    # So is a call with more requests x kv heads than the built-in counters (4096): from its sizes
    # alone, before anything is read.  (Such a call also outgrows the scratch array, whichever
    # head size and split count it has; either refusal is a refusal.)
    code = fn(qkv.data_ptr(), qkv.stride(0), got.data_ptr(), got.stride(0), cache.data_ptr(), pages, None, 4097,
              info.data_ptr(), table.data_ptr(), table.stride(0), page, Hq, 1, 16, 0, scale, 64, 1,
              status.data_ptr(), stream)
    assert code != 0 and "built-in" in lib.mlr_last_error().decode()
