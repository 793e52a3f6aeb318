"""The engine at the layer sizes that are measured: Qwen3-0.6B, 8B and 32B widths, head
counts and feed-forward widths, two layers each, seeded random weights made on the device.

The tiny models never reach the kernels' schedules for real widths: K cut into nine ranges
whose partial sums the next norm adds, the two-SM gated product with its default threshold,
the vendor library's products with the add in their epilogue, key splits of 4 to 32 under
CUDA graphs that were planned for a context bucket's bound, decode batches of more than 8
rows.  Here every one of them runs, with the default routing, and the logits are compared
  * float32 engine  vs  the plain implementation in float64 (dense attention), 2e-4;
  * the four ways of cutting in float32  vs  each other, bit for bit;
  * bfloat16 engine vs  the same truth, by relative RMSE / largest difference / cosine per row.
The reference does this on its real model against its own CPU runtime and against llama.cpp
(tests/cuda_runtime_tests.cpp:112-151, docs/CUDA_NUMERICS.md:22-32).
"""
import pytest
import torch

import plain_dense
import trace_tools
from helpers import BF16_BOUNDS_REAL_SIZES, assert_close, assert_rows_close, random_tokens


def check(got, want, dtype, what):
    if dtype == "bfloat16":
        assert_rows_close(got, want, what, BF16_BOUNDS_REAL_SIZES)
    else:
        assert_close(got, want, dtype, what)

pytestmark = pytest.mark.gpu

BASE = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 2, "head_dim": 128,
        "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "use_sliding_window": False, "hidden_act": "silu",
        "attention_bias": False, "torch_dtype": "bfloat16"}
SIZES = {
    # Full vocabulary and a tied head where the model is small enough for the logits of every position.
    "0.6b": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072,
                 vocab_size=151936, tie_word_embeddings=True, max_position_embeddings=4096, seed=3),
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288,
               vocab_size=10007, tie_word_embeddings=False, max_position_embeddings=8448, seed=2),
    "32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                vocab_size=5003, tie_word_embeddings=False, max_position_embeddings=4096, seed=4),
}
LENGTHS = {"a": 40, "b": 300, "c": 1100, "d": 70, "e": 200}


def config_of(name):
    config = dict(BASE, **SIZES[name])
    seed = config.pop("seed")
    return config, seed


def build(name, dtype, num_pages, max_requests=4):
    from mini_llm_runtime_b200.engine.loading import random_model
    from mini_llm_runtime_b200.engine.model import CacheConfig
    config, seed = config_of(name)
    return random_model(config, seed, dtype, CacheConfig(page_size=16, num_pages=num_pages, max_requests=max_requests))


def weights_of(name):
    """The tensors `random_model` makes for this seed, by checkpoint name, on the device."""
    from mini_llm_runtime_b200 import models as _models  # noqa: F401
    from mini_llm_runtime_b200.config.registry import config_from_dict, plan_for
    from mini_llm_runtime_b200.engine.structure import expected_weights
    from mini_llm_runtime_b200.weights.random_init import random_tensors
    config, seed = config_of(name)
    return random_tensors(expected_weights(plan_for(config_from_dict(config))), seed, torch.bfloat16, "cuda:0")


def truth(name, tokens, rows=None):
    config, _ = config_of(name)
    return plain_dense.forward_rows(config, weights_of(name), tokens, rows, torch.float64, "cuda:0").float()


def replay(model, trace):
    """Runs a trace of `trace_tools` through `Model.step` in this process (the same calls
    bin/trace_run makes) and returns the logits by (request, position), on the device."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    slots, position, out = {}, {}, {}
    for step in trace:
        entries = []
        for e in step["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = model.open_request()
            entries.append(StepEntry(slots[e["id"]], e["tokens"], e["want"]))
        logits = model.step(entries)
        row = 0
        for e in step["entries"]:
            start = position.get(e["id"], 0)
            for w in e["want"]:
                out[(e["id"], start + w)] = logits[row].clone()
                row += 1
            position[e["id"]] = start + len(e["tokens"])
        for k in step["end"]:
            model.close_request(slots.pop(k))
            position.pop(k)
    model.check_status()
    return out


@pytest.fixture(scope="module", params=list(SIZES))
def sized(request):
    name = request.param
    config, _ = config_of(name)
    requests = {k: random_tokens(config, n, 40 + i) for i, (k, n) in enumerate(LENGTHS.items())}
    want = {k: truth(name, t) for k, t in requests.items()}
    torch.cuda.empty_cache()
    return name, requests, want


def traces(requests):
    return {"whole": trace_tools.whole(requests), "last 32 one by one": trace_tools.last_32_one_by_one(requests),
            "portions": trace_tools.portions(requests, sizes=(16, 7, 2, 5, 2, 33, 1, 3, 2, 64, 300, 130)),
            "mixed": trace_tools.mixed(requests, seed=5, live_limit=3)}


def test_four_cuts_in_float32_and_bfloat16(sized):
    """Requests of 40 to 1100 tokens: whole, the last 32 tokens one by one (from CUDA
    graphs after the second), in portions of changing size, and mixed with so few pages that
    they are used again."""
    name, requests, want = sized
    cuts = traces(requests)
    mixed_pages = trace_tools.max_live_tokens(cuts["mixed"]) // 16
    assert mixed_pages < sum(trace_tools.round64(n) for n in LENGTHS.values()) // 16, "the mixed trace must reuse pages"
    results = {}
    for dtype in ("float32", "bfloat16"):
        for cut, trace in cuts.items():
            pages = mixed_pages if cut == "mixed" else trace_tools.max_live_tokens(trace) // 16
            model = build(name, dtype, pages)
            logits = replay(model, trace)
            if cut == "last 32 one by one":
                assert model._graphs, "single-token steps did not reach the CUDA graphs"
            for k, tokens in requests.items():
                got = trace_tools.stack(logits, k, len(tokens))
                check(got, want[k], dtype, f"{name} {dtype} {cut} request {k}")
                results[(dtype, cut, k)] = got
            del model, logits
            torch.cuda.empty_cache()
    for cut in cuts:
        for k in requests:
            assert torch.equal(results[("float32", cut, k)], results[("float32", "whole", k)]), \
                f"{name}: float32 logits of request {k} depend on the cut ({cut})"


def test_decode_batch_of_twelve(sized):
    """Twelve requests decode together: more rows than the few-row products take, so every
    product of the step goes the other way; three steps, so the third comes from a graph."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    name, requests, want = sized
    tokens = requests["b"]
    for dtype in ("float32", "bfloat16"):
        model = build(name, dtype, num_pages=12 * 4, max_requests=12)
        slots = [model.open_request() for _ in range(12)]
        model.step([StepEntry(s, tokens[:20 + i], []) for i, s in enumerate(slots)])
        for step in range(3):
            logits = model.step([StepEntry(s, [tokens[20 + i + step]], [0]) for i, s in enumerate(slots)])
            for i in range(12):
                check(logits[i:i + 1], want["b"][20 + i + step:21 + i + step], dtype,
                             f"{name} {dtype} request {i} of twelve, step {step}")
        model.check_status()
        assert bool(model._graphs)
        del model
        torch.cuda.empty_cache()


def test_decoding_at_context_8192():
    """One request of the 8B sizes: 8192 tokens in portions of 2048, then 32 single tokens
    whose attention runs as 4 to 32 key splits, from the third step on out of a CUDA graph
    planned for the context bucket's bound.  Logits are asked for at the edges of the portions
    and at every decoded token."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    name = "8b"
    config, _ = config_of(name)
    total = 8192 + 32
    tokens = random_tokens(config, total, 77)
    edges = [0, 1, 15, 16, 2046, 2047]
    wanted = [p * 2048 + e for p in range(4) for e in edges] + list(range(8192, total))
    want = truth(name, tokens, wanted)
    torch.cuda.empty_cache()
    for dtype in ("float32", "bfloat16"):
        model = build(name, dtype, num_pages=total // 16 + 1, max_requests=1)
        slot = model.open_request()
        rows = [model.step([StepEntry(slot, tokens[p * 2048:(p + 1) * 2048], edges)]).clone() for p in range(4)]
        rows += [model.step([StepEntry(slot, [tokens[p]], [0])]).clone() for p in range(8192, total)]
        model.check_status()
        assert model._graphs
        got = torch.cat(rows)
        check(got, want, dtype, f"8b {dtype} at context 8192")
        del model
        torch.cuda.empty_cache()
