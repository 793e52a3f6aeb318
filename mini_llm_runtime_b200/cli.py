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
Options are matched exactly; a duplicate, an unknown name, a missing value or a number
outside its range is an error, worded as the reference words it (apps/options.h:12-62).
"""
from __future__ import annotations

import json
import math
import sys
import time
from dataclasses import dataclass
from typing import Dict, List, Sequence, Tuple

USAGE = ("mini-llm --model DIR [--prompt-ids 1,2,3] [--tokens 32] [--temperature 0] [--seed 0]\n"
         "         [--context N] [--chunk 32] [--batch 256] [--sequences 4] [--page-size 16]\n"
         "         [--dtype bfloat16|float32] [--policy mixed|prefill_first] [--device 0] [--ignore-eos]\n"
         "         [--random-weights SEED --config CONFIG.json] [--output FILE] [--inspect]\n")


class UsageError(ValueError):
    """A command line this program refuses; the message is what the user sees."""


@dataclass(frozen=True)
class _Option:
    """One option of the table below: how its value is read and which values it may take.
    `kind` is "flag" (no value), "text", "choice" (one of `choices`), "int" or "float" (within
    [low, high]; `low` / `high` may name another option whose value is the bound)."""
    kind: str
    default: object = None
    low: object = None
    high: object = None
    choices: Tuple[str, ...] = ()


OPTIONS: Dict[str, _Option] = {
    "--model": _Option("text"),
    "--prompt-ids": _Option("text", "1,2,3,4,5,6,7,8"),
    "--tokens": _Option("int", 32, 1, 4096),
    "--temperature": _Option("float", 0.0, 0.0, 100.0),
    "--seed": _Option("int", 0, 0, 2**63 - 1),
    "--context": _Option("int", 2048, 16, 1 << 20),
    "--sequences": _Option("int", 4, 1, 128),
    "--batch": _Option("int", 256, "--sequences", 1 << 20),
    "--chunk": _Option("int", 32, 1, "--batch"),
    "--page-size": _Option("int", 16, 1, 64),
    "--dtype": _Option("choice", "bfloat16", choices=("bfloat16", "float32")),
    "--policy": _Option("choice", "mixed", choices=("mixed", "prefill_first")),
    "--device": _Option("int", 0, 0, 1023),
    "--random-weights": _Option("int", None, 0, 2**31 - 1),
    "--config": _Option("text"),
    "--output": _Option("text"),
    "--help": _Option("flag", False),
    "--ignore-eos": _Option("flag", False),
    "--inspect": _Option("flag", False),
}


def _pair_up(argv: Sequence[str]) -> Dict[str, str]:
    """The raw text of every option given, each at most once (the reference's parser has the
    same three refusals and wording, apps/options.h:17-27)."""
    given: Dict[str, str] = {}
    words = iter(argv)
    for word in words:
        option = OPTIONS.get(word)
        if word in given:
            raise UsageError(f"duplicate option: {word}")
        value = "" if option is not None and option.kind == "flag" else next(words, None)
        if option is None or value is None:
            raise UsageError(f"unknown option or missing value: {word}")
        given[word] = value
    return given


def parse_options(argv: Sequence[str]) -> Dict[str, object]:
    """Typed values by option name (defaults filled in), and under "given" the set of names
    that stood on the command line.  Numbers outside their range are refused by name."""
    given = _pair_up(argv)
    values: Dict[str, object] = {"given": set(given)}
    for name, option in OPTIONS.items():     # table order: an option used as a bound comes before its user
        if option.kind == "flag":
            values[name] = name in given
            continue
        if name not in given:
            values[name] = option.default
            continue
        text = given[name]
        if option.kind == "text":
            values[name] = text
        elif option.kind == "choice":
            if text not in option.choices:
                raise UsageError(f"{name} must be " + " or ".join(option.choices))
            values[name] = text
        else:
            label = "integer" if option.kind == "int" else "number"
            bound = lambda b: values[b] if isinstance(b, str) else b
            try:
                number = int(text, 10) if option.kind == "int" else float(text)
            except ValueError:
                number = None
            if number is None or not math.isfinite(number) or not bound(option.low) <= number <= bound(option.high):
                raise UsageError(f"out-of-range {label}: {name}")
            values[name] = number
    return values


def parse_ids(text: str) -> List[int]:
    try:
        ids = [int(t, 10) for t in text.split(",") if t.strip() != ""]
    except ValueError:
        raise ValueError("--prompt-ids must be comma-separated integers") from None
    if not ids:
        raise ValueError("--prompt-ids is empty")
    return ids


def emit(report: dict, output_file) -> int:
    text = json.dumps(report, indent=2)
    print(text)
    if output_file:
        with open(output_file, "w", encoding="utf-8") as f:
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
    from .weights.safetensors_io import open_model_files

    config = config_from_dir(model_dir)
    plan = plan_for(config)
    files = open_model_files(model_dir)          # one file, or the shards an index names
    stored = [name for f in files for name in f.names()]
    expected = set(expected_weights(plan))
    redundant = {name for name, twin in plan.redundant_tensors if twin in expected}
    dtypes = sorted({str(f.dtype(name)).replace("torch.", "") for f in files for name in f.names()})
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as f:
        raw = json.load(f)
    keys = ("hidden_size", "num_hidden_layers", "num_attention_heads", "num_key_value_heads", "head_dim",
            "intermediate_size", "vocab_size", "max_position_embeddings", "rms_norm_eps", "rope_theta",
            "tie_word_embeddings", "use_sliding_window", "sliding_window", "max_window_layers")
    windows = sorted({str(layer.mixer.params.get("window")) for layer in plan.layers})
    return {"container": "safetensors", "files": len(files), "bytes": sum(os.path.getsize(f.path) for f in files),
            "tensors": len(stored), "stored_dtypes": dtypes,
            "architecture": plan.architecture, "dimensions": {k: raw[k] for k in keys if k in raw},
            "layers": len(plan.layers), "runs": len(plan.schedule), "windows": windows,
            "missing_tensors": sorted(expected - set(stored)), "unexpected_tensors": sorted(set(stored) - expected - redundant)}


def main(argv: Sequence[str]) -> int:
    try:
        opt = parse_options(argv)
        if opt["--help"] or opt["--model"] is None:
            sys.stdout.write(USAGE)
            return 0 if opt["--help"] else 1
        model_dir = opt["--model"]
        if opt["--random-weights"] is not None:
            if opt["--config"] is None:
                raise UsageError("--random-weights needs --config CONFIG.json")
            from .weights.random_init import write_random_model
            with open(opt["--config"], "r", encoding="utf-8") as f:
                write_random_model(model_dir, json.load(f), opt["--random-weights"])
        if opt["--inspect"]:
            return emit(inspect(model_dir), opt["--output"])
        dtype, policy = opt["--dtype"], opt["--policy"]
        prompt = parse_ids(opt["--prompt-ids"])
        count, sequences, page, context = opt["--tokens"], opt["--sequences"], opt["--page-size"], opt["--context"]
        batch, chunk = opt["--batch"], min(opt["--chunk"], opt["--batch"])
        temperature, seed, device = opt["--temperature"], opt["--seed"], opt["--device"]
        if len(prompt) + count > context:
            raise UsageError("prompt and output exceed the context budget")

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
        engine.submit(prompt, SamplingParams(count, temperature, seed, opt["--ignore-eos"]))
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
            "used_kv_pages_before_release": peak_pages, "used_kv_pages_after_release": used_after}, opt["--output"])
    except Exception as error:  # the reference prints the message and exits 1 (apps/mini_main.cpp:132-135)
        sys.stderr.write(f"mini-llm: {error}\n")
        return 1
