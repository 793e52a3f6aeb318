"""Each request alone and whole: the engine's logits at every position against the
plain implementation, in float32 and in bfloat16."""
import pytest
import torch

import plain_qwen3
from helpers import assert_close, engine_model, random_tokens, run_portions, run_whole, tiny_folder

pytestmark = pytest.mark.gpu

CASES = [("tiny_a", 0, 100), ("tiny_b", 1, 150), ("tiny_c", 2, 200)]


@pytest.fixture(scope="module", params=CASES, ids=[c[0] for c in CASES])
def case(request, tmp_path_factory):
    name, seed, length = request.param
    folder, config, weights = tiny_folder(tmp_path_factory, name, seed)
    tokens = random_tokens(config, length, seed + 100)
    want = plain_qwen3.forward(config, weights, tokens)
    return folder, config, tokens, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt(case, dtype):
    folder, config, tokens, want = case
    model = engine_model(folder, dtype, num_pages=32)
    assert_close(run_whole(model, tokens), want, dtype, "whole prompt")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens(case, dtype):
    folder, config, tokens, want = case
    model = engine_model(folder, dtype, num_pages=32)
    for n in (1, 2, 3):
        assert_close(run_whole(model, tokens[:n]), want[:n], dtype, f"first {n} tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_one_by_one(case, dtype):
    folder, config, tokens, want = case
    model = engine_model(folder, dtype, num_pages=32)
    got = run_portions(model, tokens, [len(tokens) - 32, 1])
    assert_close(got, want, dtype, "prompt then 32 single tokens")
