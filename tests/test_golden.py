"""The plain implementation against lilong555/mini-llm-runtime's own CPU forward pass.

`tests/golden/*.reference_logits.f32` were made once by
`tests/golden/make_reference_golden.py`, which compiles the reference's
src/minillm/runtime.cpp (and what it needs) unchanged and runs it on tiny random
models.  The reference keeps keys and values in float16 (src/minillm/paged_kv.cpp:85-98)
while the plain implementation keeps them in float32; with logits of order 1 that
rounding is worth a few 1e-4, which is what the bound below allows.
"""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3
import tiny_models

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_plain_implementation_matches_the_reference_runtime(name):
    with open(os.path.join(GOLDEN, name + ".json")) as f:
        meta = json.load(f)
    config = tiny_models.get(name)
    weights = plain_qwen3.random_weights(config, meta["weight_seed"])
    want = torch.from_numpy(np.fromfile(os.path.join(GOLDEN, name + ".reference_logits.f32"), dtype="<f4")
                            .reshape(len(meta["tokens"]), meta["vocab"]).copy())
    got = plain_qwen3.forward(config, weights, meta["tokens"])
    diff = (got - want).abs()
    assert diff.max() < 1e-3, f"max abs diff {diff.max():.3e}"
    assert torch.sqrt((diff ** 2).mean()) < 2e-4
    assert (got.argmax(-1) == want.argmax(-1)).float().mean() > 0.95
    cosine = torch.nn.functional.cosine_similarity(got, want, dim=-1).min()
    assert cosine > 0.99999
