"""A small, fixed workload for profilers: a few decode steps or one prefill of the
Qwen3-8B layer sizes with few layers, bracketed by cudaProfilerStart/Stop.

    python -m mini_llm_runtime_b200.profiling decode  [--layers 2] [--batch 8] [--context 8192] [--steps 2]
    python -m mini_llm_runtime_b200.profiling prefill [--layers 2] [--tokens 2048] [--mma-sync-attention]

Meant to run under `ncu --profile-from-start off ...`: with two layers it holds about
4 GB on the device and launches a few dozen kernels inside the profiled region, so a
capture ends by itself within a minute or two.  Run it once without the profiler first;
it prints the time per step it measured with CUDA events.
"""
from __future__ import annotations

import argparse

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
    ap.add_argument("mode", choices=["decode", "prefill"])
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--mma-sync-attention", action="store_true",
                    help="prompt attention on the mma.sync kernel instead of the tcgen05 one")
    args = ap.parse_args()

    from .engine.loading import random_model
    from .engine.model import CacheConfig, StepEntry
    from .sampling.sampler import Sampler

    cfg = dict(QWEN3_8B, num_hidden_layers=args.layers)
    length = args.context if args.mode == "decode" else args.tokens
    batch = args.batch if args.mode == "decode" else 1
    model = random_model(cfg, 2, "bfloat16", CacheConfig(page_size=args.page_size, num_pages=batch * (length // args.page_size + 8),
                                                         max_requests=batch, max_model_len=length + 64, fill_nan=False))
    model.use_graphs = not args.no_graphs
    model.rt.tcgen05_attention = not args.mma_sync_attention
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


if __name__ == "__main__":
    raise SystemExit(main())
