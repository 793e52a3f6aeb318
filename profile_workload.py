"""A small, fixed workload for profilers: a few decode steps or one prefill of the
Qwen3-8B layer sizes with few layers, bracketed by cudaProfilerStart/Stop.

    python profile_workload.py decode  [--layers 2] [--batch 8] [--context 8192] [--steps 2]
    python profile_workload.py prefill [--layers 2] [--tokens 2048] [--mma-sync-attention]
    python profile_workload.py attention [--page-size 64]
    python profile_workload.py products  [--tokens 2048]

`attention` times the two bfloat16 attention kernels alone (CUDA events, no model) over a
range of prompt lengths, contexts, batch sizes and head sizes and prints two tables.
`products` does the same for the matrix products of a prompt portion (`--tokens` rows) at
the 8B layer sizes: the two-SM tcgen05 kernel with each epilogue, the one-block kernel and
the vendor library, each timed over a loop with the L2 flushed between launches; the profiled
region holds three launches of the two-SM kernel with the gate epilogue.

Meant to run under ncu, which must be given `--clock-control none` every time (its default
locks the GPU's clocks, and the lock can outlast the process on a shared GPU):

    ncu --clock-control none --profile-from-start off --metrics gpu__time_duration.sum \
        --csv --log-file launches.csv python profile_workload.py decode          (every launch of the region)
    ncu --clock-control none --profile-from-start off --set full -k regex:<one kernel> -c 2 \
        -o report python profile_workload.py decode                             (one kernel in depth)

With two layers it holds about 4 GB on the device and launches a few dozen kernels inside
the profiled region, so a capture ends by itself within a minute or two.  Run the same
command once without the profiler first; it prints the time per step measured with CUDA events.
This file is a measurement tool beside `bench.py`; nothing in the package imports it.
"""
from __future__ import annotations

import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

import torch

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 4096, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "use_sliding_window": False, "hidden_act": "silu", "attention_bias": False,
    "torch_dtype": "bfloat16",
}


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("mode", choices=["decode", "prefill", "attention", "products"])
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--gemv-rows", type=int, default=-1,
                    help="up to how many rows a product takes the CUDA-core pass over the weights (default: the runtime's setting)")
    ap.add_argument("--mma-sync-attention", action="store_true",
                    help="prompt attention on the mma.sync kernel instead of the tcgen05 one")
    args = ap.parse_args()

    if args.mode == "attention":
        return attention_tables(args.page_size if args.page_size != 16 else 64)

    if args.mode == "products":
        return product_table(args.tokens)

    from mini_llm_runtime_b200.engine.loading import random_model
    from mini_llm_runtime_b200.engine.model import CacheConfig, StepEntry
    from mini_llm_runtime_b200.sampling.sampler import Sampler

    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    length = args.context if args.mode == "decode" else args.tokens
    batch = args.batch if args.mode == "decode" else 1
    model = random_model(cfg, 2, "bfloat16", CacheConfig(page_size=args.page_size, num_pages=batch * (length // args.page_size + 8),
                                                         max_requests=batch, max_model_len=length + 64, fill_nan=False))
    model.use_graphs = not args.no_graphs
    model.rt.tcgen05_attention = not args.mma_sync_attention
    if args.gemv_rows >= 0:
        model.rt.gemv_rows = args.gemv_rows
    g = torch.Generator().manual_seed(0)
    tokens = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if args.mode == "decode":
        sampler = Sampler(model.rt.device, model.status)
        slots = [model.open_request() for _ in range(batch)]
        for s in slots:
            prompt = tokens(length - 1)
            for p in range(0, len(prompt), 2048):
                model.step([StepEntry(s, prompt[p:p + 2048], [])])
        ids = torch.zeros(batch, dtype=torch.int32, device=model.rt.device)
        entries = [StepEntry(s, [0], [0]) for s in slots]

        def step():
            nonlocal ids
            ids = sampler.sample(model.step(entries, device_tokens=ids))

        for _ in range(3):
            step()
        torch.cuda.synchronize()
        start.record()
        for _ in range(10):
            step()
        end.record()
        torch.cuda.synchronize()
        print(f"decode: {start.elapsed_time(end) / 10:.3f} ms per step ({args.layers} layers, batch {batch}, context {length})")
        torch.cuda.cudart().cudaProfilerStart()
        for _ in range(args.steps):
            step()
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
    else:
        prompt = tokens(length)

        def prefill():
            slot = model.open_request()
            model.step([StepEntry(slot, prompt, [length - 1])])
            model.close_request(slot)

        for _ in range(2):
            prefill()
        torch.cuda.synchronize()
        start.record()
        for _ in range(3):
            prefill()
        end.record()
        torch.cuda.synchronize()
        print(f"prefill: {start.elapsed_time(end) / 3:.3f} ms for {length} tokens ({args.layers} layers)")
        torch.cuda.cudart().cudaProfilerStart()
        prefill()
        torch.cuda.synchronize()
        torch.cuda.cudart().cudaProfilerStop()
    model.check_status()
    return 0


def product_table(rows: int) -> int:
    """The products of one layer of the 8B sizes for `rows` tokens, each kernel alone: median
    of 20 launches after 3, a 256 MB buffer written between launches so that operands come
    from DRAM."""
    from mini_llm_runtime_b200.ops import functions as F
    dev = "cuda:0"
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn, reps=20):
        for _ in range(3):
            fn()
        times = []
        for _ in range(reps):
            flush.zero_()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(end) * 1e3)
        return sorted(times)[len(times) // 2]

    H, I = QWEN3_8B["hidden_size"], QWEN3_8B["intermediate_size"]
    qkv = (QWEN3_8B["num_attention_heads"] + 2 * QWEN3_8B["num_key_value_heads"]) * QWEN3_8B["head_dim"]
    gen = torch.Generator(device=dev).manual_seed(0)
    print(f"| product ({rows} rows) | library | one-block tcgen05 | two-SM tcgen05 | two-SM TFLOP/s |")
    print("| --- | ---: | ---: | ---: | ---: |")
    gated = None
    for name, N, K in (("q/k/v", qkv, H), ("o_proj", H, QWEN3_8B["num_attention_heads"] * QWEN3_8B["head_dim"]),
                       ("gate/up", 2 * I, H), ("down_proj", H, I)):
        x = torch.randn(rows, K, device=dev, generator=gen).bfloat16()
        w = (torch.randn(N, K, device=dev, generator=gen) * 0.02).bfloat16()
        out = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
        lib = timed(lambda: torch.mm(x, w.t(), out=out))
        one = timed(lambda: F.gemm_bf16_tcgen05(x, w, out, status))
        pair = timed(lambda: F.gemm_bf16_tcgen05_pair(x, w, out, status, "bf16"))
        print(f"| {name} {N} x {K}, bfloat16 out | {lib:.1f} | {one:.1f} | {pair:.1f} | {2 * rows * N * K / pair / 1e6:.0f} |")
        if name in ("o_proj", "down_proj"):
            h = torch.zeros(rows, N, device=dev)
            lib = timed(lambda: torch.addmm(h, x, w.t(), out_dtype=torch.float32, out=h))
            pair = timed(lambda: F.gemm_bf16_tcgen05_pair(x, w, h, status, "add_f32"))
            print(f"| {name}, added into the float32 stream | {lib:.1f} | | {pair:.1f} | {2 * rows * N * K / pair / 1e6:.0f} |")
        if name == "gate/up":
            stacked = F.interleave_gate_up(w[:I], w[I:])
            act = torch.empty(rows, I, dtype=torch.bfloat16, device=dev)

            def library_then_gate():
                torch.mm(x, stacked.t(), out=out)
                F.swiglu(out, act, F.GATE_BLOCK)

            gated = lambda: F.gemm_bf16_tcgen05_pair(x, stacked, act, status, "silu_gate")
            lib, pair = timed(library_then_gate), timed(gated)
            print(f"| gate/up with the SiLU gate (library: product, then gate kernel) | {lib:.1f} | | {pair:.1f} | "
                  f"{2 * rows * N * K / pair / 1e6:.0f} |")
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStart()
            for _ in range(3):
                gated()
            torch.cuda.synchronize()
            torch.cuda.cudart().cudaProfilerStop()
    if status.item():
        raise RuntimeError(f"a kernel reported status {status.item()}")
    return 0


def attention_tables(page: int) -> int:
    """The prompt kernel (tcgen05) and the decode kernel (split-KV) alone, random data, pages
    in random order for decode; time per launch from CUDA events over 10 launches after 3."""
    import math

    from mini_llm_runtime_b200.engine import executor
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    from mini_llm_runtime_b200.ops import functions as F
    dev = "cuda:0"

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / reps

    def prefill(tokens, heads, kv_heads, dim, window=0, before=0):
        blocks = (before + tokens + page - 1) // page
        cache = (torch.randn(blocks, 2, kv_heads, page, dim, device=dev) * 0.5).to(torch.bfloat16)
        table = torch.arange(blocks, device=dev, dtype=torch.int32).view(1, blocks)
        info = torch.tensor([[0, tokens, before, 0]], dtype=torch.int32, device=dev)
        qkv = torch.randn(tokens, (heads + 2 * kv_heads) * dim, device=dev).to(torch.bfloat16)
        out = torch.empty(tokens, heads * dim, device=dev, dtype=torch.bfloat16)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        tiles = sorted(((0, t) for t in range(0, tokens, 128)), key=lambda x: -x[1])
        tiles = torch.tensor(tiles, dtype=torch.int32, device=dev)
        ms = timed(lambda: F.attention_prefill_tcgen05(qkv, out, cache, tiles, info, table, page, heads, kv_heads, dim, window,
                                                       1 / math.sqrt(dim), status))
        pairs = sum(min(before + t + 1, window) if window else before + t + 1 for t in range(tokens))
        print(f"| {tokens} | {before} | {heads}/{kv_heads} x {dim} | {window or '-'} | {ms * 1e3:.0f} | {4 * heads * dim * pairs / ms / 1e9:.0f} |")
        assert status.item() == 0

    def decode(batch, context, heads, kv_heads, dim):
        blocks = (context + page - 1) // page
        cache = (torch.randn(batch * blocks, 2, kv_heads, page, dim, device=dev) * 0.5).to(torch.bfloat16)
        table = torch.randperm(batch * blocks, device=dev).to(torch.int32).view(batch, blocks)
        info = torch.tensor([[i, 1, context - 1, i] for i in range(batch)], dtype=torch.int32, device=dev)
        qkv = torch.randn(batch, (heads + 2 * kv_heads) * dim, device=dev).to(torch.bfloat16)
        out = torch.empty(batch, heads * dim, device=dev, dtype=torch.bfloat16)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        planned = executor.plan_attention((heads // kv_heads, kv_heads, 0, 1, dim, 1), [(context - 1, 1)] * batch, 0, sms)
        chunk, splits = planned["chunk"], planned["max_splits"]
        partial = torch.empty(max(1, F.attention_decode_scratch_floats(batch, kv_heads, dim, splits)), device=dev)
        counters = torch.zeros(batch * kv_heads, dtype=torch.int32, device=dev)
        ms = timed(lambda: F.attention_decode_bf16(qkv, out, cache, None, batch, info, table, page, heads, kv_heads, dim, 0,
                                                   1 / math.sqrt(dim), chunk, splits, partial, status, counters=counters))
        gb = batch * context * kv_heads * dim * 2 * 2 / 1e9
        print(f"| {batch} | {context} | {heads}/{kv_heads} x {dim} | {splits} x {chunk} | {ms * 1e3:.1f} | {gb / ms:.2f} |")
        assert status.item() == 0

    print(f"pages of {page} tokens\n\n| prompt tokens | context before | heads x size | window | µs | TFLOP/s (causal) |\n| ---: | ---: | --- | ---: | ---: | ---: |")
    for tokens in (512, 1024, 2048, 4096, 8192, 16384, 32768):
        prefill(tokens, 32, 8, 128)
    prefill(2048, 32, 8, 128, before=30720)
    prefill(2048, 32, 8, 128, window=4096, before=30720)
    for tokens in (2048, 8192):
        prefill(tokens, 16, 4, 64)
    print("\n| requests | context | heads x size | splits x keys | µs | TB/s of cache bytes |\n| ---: | ---: | --- | --- | ---: | ---: |")
    for batch, context in ((1, 1024), (1, 8192), (1, 32768), (1, 131072), (8, 1024), (8, 4096), (8, 8192), (8, 32768), (64, 1024),
                           (64, 4096), (64, 8192), (64, 32768), (256, 2048)):
        decode(batch, context, 32, 8, 128)
    for batch, context in ((8, 8192), (64, 8192)):
        decode(batch, context, 16, 4, 64)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
