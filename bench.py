#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, one JSON line.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The default run is the Qwen3-8B layer sizes (36 layers, width 4096, 32/8 heads of
128, feed-forward 12288, vocabulary 151936, untied head) with seeded random weights
in bfloat16, pages of 16 tokens, 8 requests each holding 8192 tokens of context.
A step is one decode step of the whole batch.

  value      decoded tokens per second, timed on the device with CUDA events around K
             steps whose sampled tokens stay on the device
  e2e        the same through the public entry point (Engine.submit / Engine.step):
             every step its inputs (token slots, positions, block tables) go host ->
             device from pinned memory and its sampled ids come device -> host; the
             engine launches the next decode step before it reads the last one back,
             feeding it the ids on the device, so its bookkeeping runs beside the GPU
  prefill    one request of 2048 tokens in one step: tokens/s, ms, and flops / time /
             bf16 peak
  roofline   bytes a decode step must read (every weight once plus the cache of the
             live requests) / step time, against the HBM peak
  points     decode tokens/s at batch 1 and 64 (same context), and at batch 1/8/64
             with 2048 tokens of context
  checked    before anything is timed, the timed configuration cut to two layers (same seed, so
             the same tensors) runs its prompts and first decode steps in bfloat16 and in true
             float32, and the logits and greedy ids of the two must agree (relative RMSE, largest
             difference and cosine per row); if they do not, no number is printed (`--no-check`
             skips this)
  steady_state   the timed decode steps must not grow a buffer of the step executor nor make the
             allocator ask the driver for memory; weights are never copied again and no logits
             leave the device
  reference_point   the engine at the configuration the reference arm runs (Qwen3-0.6B sizes,
             batch 4, context 2048; bfloat16 here, float32 there), for a like-for-like ratio

Peaks come from MEASURED_PEAKS.json beside this file when it exists, else from the
fallback figures of an earlier measurement on the same pool (6.65 TB/s, 1.59 PFLOP/s).
Prompts are seeded uniform-random token ids; weights are random; no dataset is used.
The timed steps read 15 GB of weights each, far more than the 126 MB L2, so no
explicit L2 flush is needed between them.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": 4096, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 12288,
    "vocab_size": 151936, "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "tie_word_embeddings": False, "use_sliding_window": False, "hidden_act": "silu", "attention_bias": False,
    "torch_dtype": "bfloat16",
}
# The two other sizes the baseline names: (configuration, weights seed, context, batch of the headline, largest batch).
QWEN3_06B = dict(QWEN3_8B, hidden_size=1024, num_hidden_layers=28, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True)
QWEN3_32B = dict(QWEN3_8B, hidden_size=5120, num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8,
                 intermediate_size=25600)
MODELS = {"qwen3-8b": (QWEN3_8B, 2, 8192, 64), "qwen3-0.6b": (QWEN3_06B, 3, 4096, 64), "qwen3-32b": (QWEN3_32B, 4, 4096, 32)}
QUICK = dict(QWEN3_8B, hidden_size=512, num_hidden_layers=4, num_attention_heads=8, num_key_value_heads=2,
             head_dim=64, intermediate_size=1024, vocab_size=4099, max_position_embeddings=4096)


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if os.path.exists(path):
        try:
            with open(path) as f:
                data = json.load(f)
            out["hbm_gbs"] = float(data.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(data.get("bf16_tflops", out["bf16_tflops"]))
            out["source"] = "measured"
        except (OSError, ValueError):
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, device_index: int = 0):
        self.lines, self.proc, self.device_index = [], None, device_index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.device_index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self):
        clocks, maxes, reasons = [], [], set()
        for line in self.lines:
            cells = [c.strip() for c in line.split(",")]
            if len(cells) < 6:
                continue
            try:
                clocks.append(int(cells[0]))
                maxes.append(int(cells[1]))
            except ValueError:
                continue
            for name, cell in zip(self.NAMES, cells[2:6]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        if not clocks:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": int(statistics.median(clocks)), "sm_max_mhz": max(maxes), "reasons": sorted(reasons),
                "samples": len(clocks)}


REFERENCE_BINARY = os.path.join(ROOT, "baseline", "_ref", "ref_bench")
# The reference's CUDA runtime takes at most 4 sequences of 2048 positions and 128 rows a step, with
# float32 products (include/minillm/cuda/runtime.h:18-23, include/minillm/cuda/kv_layout.h:29-31), and is
# written for Qwen3-0.6B: that is the configuration its arm runs.
REFERENCE_BATCH, REFERENCE_CONTEXT = 4, 2048


def reference_arm(args) -> int:
    """Runs lilong555/mini-llm-runtime's own CUDA runtime, compiled unchanged by
    `baseline/build_reference.py` into baseline/_ref/ref_bench (a driver over its public
    `CudaRuntime::forward` with stand-ins for the two classes that need llama.cpp), at the
    Qwen3-0.6B sizes with synthetic float32 weights: decode at batch 4 and context 2048, its
    limits.  That is NOT the headline's configuration (8B sizes, batch 8, context 8192), which
    the reference cannot run; `same_config` says so, and the line of `--impl ours` carries the
    engine's own figures at this configuration under `reference_point`."""
    if not os.path.exists(REFERENCE_BINARY):
        print(json.dumps({"impl": "reference",
                          "unavailable": "baseline/_ref/ref_bench is not built: run `python baseline/build_reference.py "
                                         "<checkout of lilong555/mini-llm-runtime>` (the reference is a CMake C++/CUDA project, "
                                         "`pip install` of it finds neither setup.py nor pyproject.toml)"}))
        return 0
    c = QWEN3_06B
    spec = (f"synthetic:{c['hidden_size']}:{c['num_hidden_layers']}:{c['num_attention_heads']}:{c['num_key_value_heads']}:"
            f"{c['head_dim']}:{c['intermediate_size']}:{c['vocab_size']}:{c['max_position_embeddings']}:3:1")
    steps, warmup = args.steps, max(args.warmup, 3)
    with ClockSampler() as clocks:
        done = subprocess.run([REFERENCE_BINARY, spec, str(steps), str(warmup), str(REFERENCE_CONTEXT), str(REFERENCE_BATCH)],
                              capture_output=True, text=True)
    if done.returncode != 0:
        reason = (done.stderr.strip().splitlines() or ["no message"])[-1]
        print(json.dumps({"impl": "reference", "unavailable": f"baseline/_ref/ref_bench exited {done.returncode}: {reason}"}))
        return 0
    r = json.loads(done.stdout.strip().splitlines()[-1])
    d = r["decode"]
    device_ms, wall_ms = d["device_ms"] / d["steps"], d["wall_ms"] / d["steps"]
    b1, pf = r["decode_b1"], r["prefill_128"]
    print(json.dumps({
        "metric": f"decode tok/s (Qwen3-0.6B sizes, batch {REFERENCE_BATCH}, context {REFERENCE_CONTEXT}, fp32)",
        "value": REFERENCE_BATCH / device_ms * 1e3, "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": device_ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp32",
        "data": "synthetic", "impl": "reference", "same_config": False,
        "config": {"model": "Qwen3-0.6B sizes, synthetic float32 weights", "layers": c["num_hidden_layers"],
                   "hidden": c["hidden_size"], "q_heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
                   "head_dim": c["head_dim"], "intermediate": c["intermediate_size"], "vocab": c["vocab_size"],
                   "global_batch": REFERENCE_BATCH, "seq_len": REFERENCE_CONTEXT, "parallelism": "single_gpu",
                   "limits": "the reference's own: 4 sequences, 2048 positions, 128 rows a step, float32 products",
                   "l2": "inputs>L2 (2.4 GB of float32 weights per step), no flush"},
        "clocks": clocks.summary(),
        "e2e": {"value": REFERENCE_BATCH / wall_ms * 1e3, "unit": "tokens/s", "ms_per_step": wall_ms,
                "h2d_bytes_per_step": 4 * 3 * REFERENCE_BATCH + 4 * REFERENCE_BATCH, "d2h_bytes_per_step": 4 * REFERENCE_BATCH + 8},
        "points": {"decode_b1_ctx2048": 1.0 / (b1["device_ms"] / b1["steps"]) * 1e3,
                   "prefill_128_tokens_per_s": 128.0 / (pf["device_ms"] / pf["repeats"]) * 1e3},
        "load_ms": r["load_ms"], "poisoned": r["poisoned"]}))
    return 0


# What bfloat16 may differ from float32 by at the layer sizes of real models, per row of logits and relative to
# the size of the row (tests/test_real_sizes.py measures 0.012 / 0.060 / 0.99993 against float64).
CHECK_BOUNDS = {"rmse": 0.025, "max": 0.12, "cosine": 0.99985}


def check_configuration(cfg, seed, batch, context, page, steps=3):
    """The timed configuration with two layers, in bfloat16 and in float32: prompts of `context - 1`
    tokens in portions of 2048, then `steps` decode steps that both precisions take with the float32
    path's greedy ids.  Returns a short report; raises if logits or ids disagree."""
    import torch
    from mini_llm_runtime_b200.engine.loading import random_model
    from mini_llm_runtime_b200.engine.model import CacheConfig, StepEntry
    cut = dict(cfg, num_hidden_layers=min(2, cfg["num_hidden_layers"]))
    gen = torch.Generator().manual_seed(4321)
    prompts = [torch.randint(0, cfg["vocab_size"], (context - 1,), generator=gen).tolist() for _ in range(batch)]
    first = torch.randint(0, cfg["vocab_size"], (batch,), generator=gen).tolist()
    pages = batch * ((context + steps + page) // page + 1)
    rows = {}
    for dtype in ("float32", "bfloat16"):
        model = random_model(cut, seed=seed, dtype=dtype,
                             cache=CacheConfig(page_size=page, num_pages=pages, max_requests=batch, max_model_len=context + steps + page))
        slots = [model.open_request() for _ in range(batch)]
        for slot, prompt in zip(slots, prompts):
            for pos in range(0, len(prompt), 2048):
                model.step([StepEntry(slot, prompt[pos:pos + 2048], [])])
        tokens, out = list(first), []
        for step in range(steps):
            logits = model.step([StepEntry(s, [t], [0]) for s, t in zip(slots, tokens)]).clone()
            out.append(logits)
            tokens = (rows["float32"][step] if dtype == "bfloat16" else logits).argmax(-1).tolist()
        model.check_status()
        rows[dtype] = out
        del model
        torch.cuda.empty_cache()
    worst = {"rmse": 0.0, "max": 0.0, "cosine": 1.0}
    flips = 0
    for want, got in zip(rows["float32"], rows["bfloat16"]):
        want, got = want.double(), got.double()
        size = want.pow(2).mean(-1).sqrt()
        diff = got - want
        worst["rmse"] = max(worst["rmse"], float((diff.pow(2).mean(-1).sqrt() / size).max()))
        worst["max"] = max(worst["max"], float((diff.abs().amax(-1) / size).max()))
        worst["cosine"] = min(worst["cosine"], float(((got * want).sum(-1) / (got.norm(dim=-1) * want.norm(dim=-1))).min()))
        for r in range(want.shape[0]):
            a, b = int(want[r].argmax()), int(got[r].argmax())
            if a != b:
                if float(want[r, a] - want[r, b]) > 2 * CHECK_BOUNDS["max"] * float(size[r]):
                    raise RuntimeError(f"check: bfloat16 picks token {b} where float32 picks {a}, {float(want[r, a] - want[r, b]):.4f} apart")
                flips += 1
    if worst["rmse"] > CHECK_BOUNDS["rmse"] or worst["max"] > CHECK_BOUNDS["max"] or worst["cosine"] < CHECK_BOUNDS["cosine"]:
        raise RuntimeError(f"check: bfloat16 and float32 logits disagree: {worst} against the bounds {CHECK_BOUNDS}")
    return {"layers": cut["num_hidden_layers"], "decode_steps": steps, "rows": steps * batch, "relative_rmse": round(worst["rmse"], 5),
            "relative_max": round(worst["max"], 5), "cosine": round(worst["cosine"], 7), "near_tie_flips": flips}


def matmul_params(cfg, layers):
    H, D = cfg["hidden_size"], cfg["head_dim"]
    per_layer = (cfg["num_attention_heads"] + 2 * cfg["num_key_value_heads"]) * D * H + cfg["num_attention_heads"] * D * H \
        + 3 * cfg["intermediate_size"] * H
    return per_layer * layers, cfg["vocab_size"] * H


def serving(args, cfg, model, prompt_of, gen) -> int:
    """The baseline's mixed workload: 64 requests arrive at once, prompt lengths uniform in
    [16, 2048], 256 generated tokens each, greedy, through the Python entry point (host token
    ids in and out; admission, chunked prompts beside decoding requests, pages given back)."""
    import torch
    from mini_llm_runtime_b200.engine.api import LLM
    requests, new_tokens = 64, 256
    lengths = torch.randint(16, 2049, (requests,), generator=gen).tolist()
    prompts = [prompt_of(n) for n in lengths]
    llm = LLM(model, max_batch_tokens=4096, prefill_chunk=2048)
    llm.generate(prompts[:4], max_tokens=8, ignore_eos=True)            # warm-up: kernels, graphs of small batches
    torch.cuda.synchronize()
    steps_before = llm.engine.steps
    t0 = time.perf_counter()
    results = llm.generate(prompts, max_tokens=new_tokens, ignore_eos=True)
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    assert all(len(r.token_ids) == new_tokens for r in results)
    steps = llm.engine.steps - steps_before
    print(json.dumps({
        "metric": "generated tok/s, 64 requests at once, prompts U[16, 2048], 256 tokens each, through LLM.generate",
        "value": requests * new_tokens / seconds, "unit": "tokens/s", "seconds": seconds, "steps": steps,
        "ms_per_step": seconds * 1e3 / steps, "prompt_tokens": sum(lengths),
        "all_tokens_per_s": (sum(lengths) + requests * new_tokens) / seconds,
        "model": args.model, "layers": cfg["num_hidden_layers"], "dtype": "bf16", "data": "synthetic",
        "max_requests": model.cache.max_requests, "page_size": args.page_size}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=0, help="default: the context length the baseline names for the model")
    ap.add_argument("--model", default="qwen3-8b", choices=sorted(MODELS),
                    help="layer sizes; the default is the configuration the headline is quoted on")
    ap.add_argument("--layers", type=int, default=0, help="run fewer layers than the configuration has (named in config)")
    ap.add_argument("--quick", action="store_true", help="a small model, for checking this script")
    ap.add_argument("--no-points", action="store_true")
    ap.add_argument("--serving", action="store_true",
                    help="instead of the headline: the baseline's mixed workload through LLM.generate (64 requests, prompts of "
                         "16 to 2048 random tokens, 256 generated tokens each); prints one JSON line of its own")
    ap.add_argument("--own-products", action="store_true",
                    help="every matrix product on the package's tcgen05 kernel, none on the vendor library (slower)")
    ap.add_argument("--page-size", type=int, default=16, help="tokens per cache page (the baseline's configuration has 16; 64 is a little faster)")
    ap.add_argument("--no-check", action="store_true", help="skip the agreement check of bfloat16 and float32 before the measurement")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 5:
        args.warmup = 5      # a decode shape is captured into a graph on its third step, and the first step may end a context bucket

    import torch
    from mini_llm_runtime_b200.engine.engine import Engine
    from mini_llm_runtime_b200.engine.loading import random_model
    from mini_llm_runtime_b200.engine.model import CacheConfig, StepEntry
    from mini_llm_runtime_b200.ops import native
    from mini_llm_runtime_b200.sampling.sampler import Sampler, SamplingParams

    model_cfg, weights_seed, model_context, largest_batch = MODELS[args.model]
    cfg = dict(QUICK if args.quick else model_cfg)
    args.context = args.context or model_context
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    layers = cfg["num_hidden_layers"]
    context, page = args.context, args.page_size
    horizon = args.steps + args.warmup + 8
    # The largest batch of the extra points must fit the memory beside the weights: halve it until it does.
    head_dim, kv_heads = cfg["head_dim"], cfg["num_key_value_heads"]
    cache_per_token = 2 * 2 * kv_heads * head_dim * layers
    weights_estimate = 2 * sum(matmul_params(cfg, layers)) + (0 if cfg["tie_word_embeddings"] else 2 * cfg["vocab_size"] * cfg["hidden_size"])
    room = 0.85 * torch.cuda.get_device_properties(0).total_memory - weights_estimate
    while largest_batch > args.batch and largest_batch * (context + horizon + page) * cache_per_token > room:
        largest_batch //= 2
    batches = [args.batch] if args.no_points else sorted({1, args.batch, largest_batch})
    max_batch = max(batches)
    pages = max_batch * ((context + horizon + page - 1) // page + 1)
    pk = peaks()

    checked = None
    if not args.no_check and not args.serving:
        try:
            checked = check_configuration(cfg, weights_seed, args.batch, context, page)
        except RuntimeError as error:
            print(f"bench.py: {error}; no number is reported", file=sys.stderr)
            return 1

    torch.manual_seed(0)
    model = random_model(cfg, seed=weights_seed, dtype="bfloat16",
                         cache=CacheConfig(page_size=page, num_pages=pages, max_requests=max_batch,
                                           max_model_len=context + horizon + page, fill_nan=False))
    if args.own_products:
        model.rt.own_products_only()
    gen = torch.Generator().manual_seed(1234)
    prompt_of = lambda n: torch.randint(0, cfg["vocab_size"], (n,), generator=gen).tolist()
    if args.serving:
        return serving(args, cfg, model, prompt_of, gen)
    layer_params, head_params = matmul_params(cfg, layers)
    weight_bytes = 2 * (layer_params + head_params)
    kv_bytes_per_token = model.cache_bytes_per_token()

    def timed(fn, reps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / reps

    # ---------------------------------------------------------------- prefill of 2048 tokens
    T = 2048 if not args.quick else 512
    prompt = prompt_of(T)

    def prefill_once():
        slot = model.open_request()
        model.step([StepEntry(slot, prompt, [T - 1])])
        model.close_request(slot)

    for _ in range(3):
        prefill_once()
    prefill_ms = timed(prefill_once, 5)
    attn_flops = 4 * cfg["num_attention_heads"] * cfg["head_dim"] * (T * (T + 1) // 2) * layers
    prefill_flops = 2 * T * layer_params + 2 * head_params + attn_flops
    prefill = {"value": T / prefill_ms * 1e3, "tokens": T, "ms": prefill_ms,
               "frac": prefill_flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12)}

    # ---------------------------------------------------------------- decode, device-timed
    sampler = Sampler(model.rt.device, model.status)

    def fill(batch, ctx):
        """Opens `batch` requests and prefills ctx-1 tokens each; returns slots and the
        device tensor of their next tokens."""
        slots = [model.open_request() for _ in range(batch)]
        chunk = 2048
        last = None
        for slot in slots:
            tokens = prompt_of(ctx - 1)
            for pos in range(0, len(tokens), chunk):
                part = tokens[pos:pos + chunk]
                final = pos + chunk >= len(tokens)
                last = model.step([StepEntry(slot, part, [len(part) - 1] if final else [])])
        return slots

    steady = {"executor_buffer_growths": 0, "driver_allocations": 0, "weight_h2d_bytes": 0, "logits_d2h_bytes": 0}

    def decode_rate(batch, ctx, steps, warmup, with_clocks=False):
        slots = fill(batch, ctx)
        ids = torch.randint(0, cfg["vocab_size"], (batch,), generator=gen).to(torch.int32).to(model.rt.device)
        entries = [StepEntry(s, [0], [0]) for s in slots]

        def one_step():
            # The sampled ids stay on the device and feed the next step.
            nonlocal ids
            logits = model.step(entries, device_tokens=ids)
            ids = sampler.sample(logits)

        for _ in range(warmup):
            one_step()
        native.reset_launches()
        grown, asked = model.steady_state_allocations, torch.cuda.memory_stats().get("num_device_alloc", 0)
        if with_clocks:
            with ClockSampler() as clocks:
                ms = timed(one_step, steps)
            clock_summary = clocks.summary()
        else:
            ms, clock_summary = timed(one_step, steps), None
        launches = native.total_launches()
        # The steady-state gates of the reference's protocol (benchmarks/runtime-inputs/qwen3-cuda-v0.json:137-144).
        steady["executor_buffer_growths"] += model.steady_state_allocations - grown
        steady["driver_allocations"] += torch.cuda.memory_stats().get("num_device_alloc", 0) - asked
        for s in slots:
            model.close_request(s)
        return batch / ms * 1e3, ms, launches, clock_summary

    value, ms_per_step, launches, clocks = decode_rate(args.batch, context, args.steps, args.warmup, with_clocks=True)
    step_bytes = weight_bytes + args.batch * (context + args.warmup + args.steps // 2) * kv_bytes_per_token
    achieved = step_bytes / (ms_per_step * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]}

    points = {}
    if not args.no_points:
        short = max(4, args.steps // 4)
        for b in (1, largest_batch):
            if b != args.batch:
                points[f"decode_b{b}"] = decode_rate(b, context, short, args.warmup)[0]
        for b in (1, 8, largest_batch):
            points[f"decode_b{b}_ctx2048"] = decode_rate(b, min(2048, context), short, args.warmup)[0]

    # ---------------------------------------------------------------- end to end through the engine
    # Prompts first, then all requests decode together (policy prefill_first), so that every
    # timed step is a decode step of the whole batch.
    engine = Engine(model, max_batch_tokens=max(2048, args.batch), prefill_chunk=2048, policy="prefill_first")
    for _ in range(args.batch):
        engine.submit(prompt_of(context - 1), SamplingParams(max_tokens=horizon, ignore_eos=True))
    while any(r.prefill_remaining for r in engine.scheduler.active) or engine.scheduler.waiting:
        engine.step()
    assert all(len(r.generated) == 1 for r in engine.scheduler.active) and len(engine.scheduler.active) == args.batch
    for _ in range(args.warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        engine.step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    e2e = {"value": args.batch / e2e_ms * 1e3, "unit": "tokens/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": model.last_h2d_bytes, "d2h_bytes_per_step": 4 * (args.batch + 1)}

    if steady["executor_buffer_growths"] or steady["driver_allocations"]:
        print(f"bench.py: the timed decode steps allocated device memory ({steady}); no number is reported", file=sys.stderr)
        return 1

    # ---------------------------------------------------------------- the reference arm's configuration, on this engine
    reference_point = None
    if args.model == "qwen3-8b" and not args.quick and not args.no_points:
        del engine, model
        torch.cuda.empty_cache()
        small = dict(QWEN3_06B)
        model = random_model(small, seed=3, dtype="bfloat16",
                             cache=CacheConfig(page_size=page, num_pages=REFERENCE_BATCH * (REFERENCE_CONTEXT // page + 8),
                                               max_requests=REFERENCE_BATCH, max_model_len=REFERENCE_CONTEXT + 64, fill_nan=False))
        sampler = Sampler(model.rt.device, model.status)
        cfg_main, cfg = cfg, small
        short = max(8, args.steps // 2)
        b4 = decode_rate(REFERENCE_BATCH, REFERENCE_CONTEXT - short - args.warmup, short, args.warmup)[0]
        b1 = decode_rate(1, REFERENCE_CONTEXT - short - args.warmup, short, args.warmup)[0]
        portion = prompt_of(128)

        def portion_once():
            slot = model.open_request()
            model.step([StepEntry(slot, portion, [127])])
            model.close_request(slot)

        for _ in range(3):
            portion_once()
        reference_point = {"model": "Qwen3-0.6B sizes", "batch": REFERENCE_BATCH, "context": REFERENCE_CONTEXT, "dtype": "bf16",
                           "decode_tok_s": b4, "decode_b1_tok_s": b1, "prefill_128_tok_s": 128 / timed(portion_once, 5) * 1e3}
        cfg = cfg_main

    name = {"qwen3-8b": "Qwen3-8B", "qwen3-0.6b": "Qwen3-0.6B", "qwen3-32b": "Qwen3-32B"}[args.model]
    config = {"model": f"{name} sizes, random weights (seed {weights_seed})" if not args.quick else "quick check model",
              "layers": layers, "layers_of_model": full_layers, "hidden": cfg["hidden_size"],
              "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
              "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
              "seq_len": context, "context_len": context, "page_size": page, "prefill_tokens": T,
              "parallelism": "single_gpu", "products": "own kernel only" if args.own_products else "own kernels for steps of up to 8 rows, own kernel and vendor library above", "l2": f"inputs>L2 ({weight_bytes / 1e9:.1f} GB of weights per step), no flush",
              "weight_gb": round(weight_bytes / 1e9, 2), "kv_kb_per_token": kv_bytes_per_token / 1024}
    print(json.dumps({
        "metric": f"decode tok/s ({name} sizes, batch {args.batch}, context {context}, bf16)", "value": value, "unit": "tokens/s",
        "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
        "config": config, "clocks": clocks, "e2e": e2e, "gpu_launches": launches, "prefill": prefill,
        "roofline": roofline, "points": points, "checked": checked is not None, "check": checked, "steady_state": steady,
        "reference_point": reference_point}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
