"""Configurations drawn at random: every size and option of the architecture at values the
fixed tiny models do not have (head sizes from 16 to 256, one to eight query heads per kv head,
widths that are multiples of 8, of 2 or odd, any vocabulary, one to five layers, windows given
by `max_window_layers` or by `layer_types`).  Each one runs whole, with the last 32 tokens
one by one, in portions and mixed with few pages, in both precisions, and one long request
reaches the kernels that only prompt portions of a thousand rows take."""
from __future__ import annotations

import random

import pytest
import torch

import plain_qwen3
import trace_tools as T
from helpers import assert_close, write_model_folder

pytestmark = pytest.mark.gpu


def random_config(rng: random.Random, widths: str) -> dict:
    head_dim = rng.choice([16, 32, 48, 64, 64, 80, 96, 112, 128, 128, 160, 192, 256])
    kv_heads = rng.choice([1, 1, 2, 3, 4])
    heads = kv_heads * rng.choice([1, 2, 3, 4, 5, 7, 8])
    if widths == "of_8":
        hidden, inter = 8 * rng.randrange(4, 40), 8 * rng.randrange(8, 60)
    elif widths == "even":
        hidden, inter = 2 * rng.randrange(16, 160), 2 * rng.randrange(8, 60)
    else:
        hidden, inter = rng.randrange(33, 300), rng.randrange(33, 400)
    layers = rng.randrange(1, 6)
    config = {"architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "hidden_size": hidden,
              "num_hidden_layers": layers, "num_attention_heads": heads, "num_key_value_heads": kv_heads,
              "head_dim": head_dim, "intermediate_size": inter, "vocab_size": rng.randrange(50, 1200),
              "max_position_embeddings": 2048, "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6, 1e-4, 1e-3]),
              "rope_theta": rng.choice([10000.0, 1e6, 5e5, 777.0, 31000.0]), "tie_word_embeddings": rng.random() < 0.5,
              "hidden_act": "silu", "attention_bias": False, "torch_dtype": "bfloat16"}
    kind = rng.random()
    if kind < 0.35:
        config["use_sliding_window"] = False
    elif kind < 0.7:
        config.update(use_sliding_window=True, sliding_window=rng.choice([3, 8, 17, 40, 64, 65, 100, 128, 150, 200, 300]),
                      max_window_layers=rng.randrange(0, layers + 1))
    else:
        config.update(use_sliding_window=True, sliding_window=rng.choice([5, 16, 33, 64, 127, 129, 256]),
                      layer_types=[rng.choice(["full_attention", "sliding_attention"]) for _ in range(layers)])
    return config


def replay(folder: str, dtype: str, trace, requests, page: int):
    from mini_llm_runtime_b200.engine.loading import load_model
    from mini_llm_runtime_b200.engine.model import CacheConfig, StepEntry
    need = T.max_live_tokens(trace)
    pages = (need + page - 1) // page + (4 if page == 64 else 0)
    model = load_model(folder, dtype, CacheConfig(page_size=page, num_pages=pages, max_requests=4))
    slots, got = {}, {k: [] for k in requests}
    for step in trace:
        entries = []
        for e in step["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = model.open_request()
            entries.append(StepEntry(slots[e["id"]], e["tokens"], e["want"]))
        out, at = model.step(entries).float().cpu(), 0
        for e in step["entries"]:
            got[e["id"]].append(out[at:at + len(e["want"])])
            at += len(e["want"])
        for k in step["end"]:
            model.close_request(slots.pop(k))
    model.check_status()
    return {k: torch.cat(v) for k, v in got.items() if v}


@pytest.mark.parametrize("seed,widths", [(77003, "of_8"), (77011, "of_8"), (77021, "of_8"), (77104, "even"), (77207, "any")])
def test_a_random_configuration_in_every_way_of_cutting(tmp_path_factory, seed, widths):
    rng = random.Random(seed)
    config = random_config(rng, widths)
    weights = plain_qwen3.random_weights(config, seed % 1000)
    folder = str(tmp_path_factory.mktemp(f"random_{seed}"))
    write_model_folder(folder, config, weights)
    draw = lambda n: [rng.randrange(config["vocab_size"]) for _ in range(n)]
    requests = {f"r{i}": draw(rng.choice([rng.randrange(2, 40), rng.randrange(40, 200), rng.randrange(200, 500)]))
                for i in range(4)}
    requests["long"] = draw(rng.randrange(1024, 1300))
    want = {k: plain_qwen3.forward(config, weights, t) for k, t in requests.items()}
    short = {k: v for k, v in requests.items() if k != "long"}
    traces = {"whole": (T.whole(requests), 16), "last 32": (T.last_32_one_by_one(short), 16),
              "portions": (T.portions(short), 16), "large portions": (T.portions({"long": requests["long"]}, (1030, 64, 2)), 16),
              "mixed": (T.mixed(short, seed=seed), 16), "mixed, pages of 64": (T.mixed(short, seed=seed + 1), 64)}
    for dtype in ("float32", "bfloat16"):
        for name, (trace, page) in traces.items():
            got = replay(folder, dtype, trace, requests, page)
            for k, logits in got.items():
                assert_close(logits, want[k], dtype, f"{config} {dtype} {name} {k}")
