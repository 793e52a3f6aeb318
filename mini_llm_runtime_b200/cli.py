"""Command line in the manner of the reference's `mini-llm` (apps/mini_main.cpp:19-27,
:71-131) and `mini-cuda-llm` (apps/cuda_main.cpp:18-26): prompt in, a JSON report with
the generated token ids and timings out.

    mini-llm --model DIR [--prompt-ids 1,2,3] [--tokens 32] [--temperature 0]
             [--seed 0] [--context N] [--chunk 32] [--batch 256] [--sequences 4]
             [--page-size 16] [--dtype bfloat16|float32] [--device 0] [--ignore-eos]
    mini-llm --model DIR --random-weights SEED --config CONFIG.json   (writes DIR first)
    mini-llm --model DIR --inspect             (what the folder holds; needs no GPU)

Names and meanings follow the reference where it has them: --model, --tokens [1,4096],
--context (cache tokens), --chunk (prompt portion per step), --batch (tokens per
step), --sequences (request slots), --device, --ignore-eos, --inspect (container and
dimensions, apps/mini_main.cpp:54-71), --output FILE (the report also goes to a file,
apps/cuda_main.cpp:18-26).  The reference takes text
(--prompt) and tokenises it with llama.cpp; this engine takes ids (--prompt-ids).
--temperature, --seed, --dtype, --page-size and --random-weights are additions.
Options are matched exactly; a duplicate, an unknown name or a missing value is an
error (apps/options.h:12-62).
"""
from __future__ import annotations

import json
import math
import sys
import time
from typing import Dict, List, Sequence

VALUES = {"--model", "--prompt-ids", "--tokens", "--temperature", "--seed", "--context", "--chunk", "--batch",
          "--sequences", "--page-size", "--dtype", "--device", "--random-weights", "--config", "--policy", "--output"}
FLAGS = {"--help", "--ignore-eos", "--inspect"}

USAGE = ("mini-llm --model DIR [--prompt-ids 1,2,3] [--tokens 32] [--temperature 0] [--seed 0]\n"
         "         [--context N] [--chunk 32] [--batch 256] [--sequences 4] [--page-size 16]\n"
         "         [--dtype bfloat16|float32] [--policy mixed|prefill_first] [--device 0] [--ignore-eos]\n"
         "         [--random-weights SEED --config CONFIG.json] [--output FILE] [--inspect]\n")


class Options:
    def __init__(self, argv: Sequence[str]):
        self.arguments: Dict[str, str] = {}
        i = 0
        while i < len(argv):
            name = argv[i]
            if name in self.arguments:
                raise ValueError(f"duplicate option: {name}")
            if name in FLAGS:
                self.arguments[name] = "true"
            elif name in VALUES and i + 1 < len(argv):
                i += 1
                self.arguments[name] = argv[i]
            else:
                raise ValueError(f"unknown option or missing value: {name}")
            i += 1

    def has(self, key: str) -> bool:
        return key in self.arguments

    def get(self, key: str, fallback: str = "") -> str:
        return self.arguments.get(key, fallback)

    def integer(self, key: str, fallback: int, minimum: int, maximum: int) -> int:
        if not self.has(key):
            return fallback
        try:
            value = int(self.get(key), 10)
        except ValueError:
            raise ValueError(f"out-of-range integer: {key}") from None
        if not minimum <= value <= maximum:
            raise ValueError(f"out-of-range integer: {key}")
        return value

    def number(self, key: str, fallback: float, minimum: float, maximum: float) -> float:
        if not self.has(key):
            return fallback
        try:
            value = float(self.get(key))
        except ValueError:
            raise ValueError(f"out-of-range number: {key}") from None
        if not math.isfinite(value) or not minimum <= value <= maximum:
            raise ValueError(f"out-of-range number: {key}")
        return value


def parse_ids(text: str) -> List[int]:
    try:
        ids = [int(t, 10) for t in text.split(",") if t.strip() != ""]
    except ValueError:
        raise ValueError("--prompt-ids must be comma-separated integers") from None
    if not ids:
        raise ValueError("--prompt-ids is empty")
    return ids


def emit(report: dict, options: "Options") -> int:
    text = json.dumps(report, indent=2)
    print(text)
    if options.has("--output"):
        with open(options.get("--output"), "w", encoding="utf-8") as f:
            f.write(text + "\n")
    return 0


def inspect(model_dir: str) -> dict:
    """What a model folder holds, read without a GPU: the container's size and tensor
    count, the architecture and the dimensions the configuration gives, the layer plan in
    short, and whether the tensors are the ones the architecture expects."""
    import os

    from . import models as _models  # noqa: F401  (registers the architectures)
    from .config.registry import config_from_dir, plan_for
    from .engine.structure import expected_weights
    from .weights.safetensors_io import SafetensorsFile

    config = config_from_dir(model_dir)
    plan = plan_for(config)
    path = os.path.join(model_dir, "model.safetensors")
    container = SafetensorsFile(path)
    stored = container.names()
    expected = set(expected_weights(plan))
    dtypes = sorted({str(container.dtype(name)).replace("torch.", "") for name in stored})
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        raw = json.load(f)
    keys = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
            "intermediate_size", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta",
            "tie_word_embeddings", "use_sliding_window", "sliding_window", "max_window_layers")
    windows = sorted({str(layer.mixer.params.get("window")) for layer in plan.layers})
    return {"container": "safetensors", "bytes": os.path.getsize(path), "tensors": len(stored), "stored_dtypes": dtypes,
            "architecture": plan.architecture, "dimensions": {k: raw[k] for k in keys if k in raw},
            "layers": len(plan.layers), "runs": len(plan.schedule), "windows": windows,
            "missing_tensors": sorted(expected - set(stored)), "unexpected_tensors": sorted(set(stored) - expected)}


def main(argv: Sequence[str]) -> int:
    try:
        options = Options(argv)
        if options.has("--help") or not options.has("--model"):
            sys.stdout.write(USAGE)
            return 0 if options.has("--help") else 1
        model_dir = options.get("--model")
        if options.has("--random-weights"):
            if not options.has("--config"):
                raise ValueError("--random-weights needs --config CONFIG.json")
            from .weights.random_init import write_random_model
            with open(options.get("--config"), "r", encoding="utf-8") as f:
                write_random_model(model_dir, json.load(f), options.integer("--random-weights", 0, 0, 2**31 - 1))
        if options.has("--inspect"):
            return emit(inspect(model_dir), options)
        dtype = options.get("--dtype", "bfloat16")
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("--dtype must be bfloat16 or float32")
        policy = options.get("--policy", "mixed")
        if policy not in ("mixed", "prefill_first"):
            raise ValueError("--policy must be mixed or prefill_first")
        prompt = parse_ids(options.get("--prompt-ids", "1,2,3,4,5,6,7,8"))
        count = options.integer("--tokens", 32, 1, 4096)
        sequences = options.integer("--sequences", 4, 1, 128)
        page = options.integer("--page-size", 16, 1, 64)
        context = options.integer("--context", 2048, 16, 1 << 20)
        batch = options.integer("--batch", 256, sequences, 1 << 20)
        chunk = options.integer("--chunk", 32, 1, batch)
        temperature = options.number("--temperature", 0.0, 0.0, 100.0)
        seed = options.integer("--seed", 0, 0, 2**63 - 1)
        device = options.integer("--device", 0, 0, 1023)
        if len(prompt) + count > context:
            raise ValueError("prompt and output exceed the context budget")

        from .engine.engine import Engine
        from .engine.loading import load_model
        from .engine.model import CacheConfig
        from .sampling.sampler import SamplingParams

        model = load_model(model_dir, dtype, None, f"cuda:{device}")
        max_len = min(context, model.plan.max_positions)
        if len(prompt) + count > max_len:
            raise ValueError(f"prompt and output exceed the model's {model.plan.max_positions} positions")
        pages = (context + page - 1) // page
        model.allocate_cache(CacheConfig(page_size=page, num_pages=pages, max_requests=sequences, max_model_len=max_len))
        engine = Engine(model, batch, chunk, policy)
        free_before = [model.cache.free_pages(g) for g in range(len(model.cache.groups))]
        start = time.perf_counter()
        engine.submit(prompt, SamplingParams(count, temperature, seed, options.has("--ignore-eos")))
        ttft_ms, peak_pages, result = 0.0, 0, None
        while engine.has_work():
            finished = engine.step()
            used = sum(b - model.cache.free_pages(g) for g, b in enumerate(free_before))
            peak_pages = max(peak_pages, used)
            active = engine.scheduler.active
            if not ttft_ms and ((active and active[0].generated) or finished):
                ttft_ms = (time.perf_counter() - start) * 1e3
            if finished:
                result = finished[0]
        elapsed = time.perf_counter() - start
        used_after = sum(b - model.cache.free_pages(g) for g, b in enumerate(free_before))
        return emit({
            "backend": "mini-llm-runtime_b200", "dtype": dtype, "token_ids": result.token_ids,
            "finish_reason": result.finish_reason, "prompt_tokens": len(prompt),
            "completion_tokens": len(result.token_ids), "ttft_ms": ttft_ms, "elapsed_s": elapsed,
            "output_tokens_per_second": len(result.token_ids) / elapsed, "steps": engine.steps,
            "used_kv_pages_before_release": peak_pages, "used_kv_pages_after_release": used_after}, options)
    except Exception as error:  # the reference prints the message and exits 1 (apps/mini_main.cpp:132-135)
        sys.stderr.write(f"mini-llm: {error}\n")
        return 1
