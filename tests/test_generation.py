"""Generation through the Python entry point and the command line against the plain
implementation: greedy, temperature, end-of-sequence, a pool that makes requests wait."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3
from helpers import assert_greedy_tokens, random_tokens, tiny_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def plain_generate(config, weights, prompt, max_tokens, temperature=0.0, seed=0, request=0, eos=(), margin=None):
    """Token by token with the whole-sequence plain forward.  With `margin`, also
    returns the smallest gap between the best and second-best logit (greedy) seen."""
    tokens, out, gap = list(prompt), [], float("inf")
    for step in range(max_tokens):
        row = plain_qwen3.forward(config, weights, tokens)[-1]
        if temperature > 0:
            token = plain_qwen3.sample_temperature(row, temperature, plain_qwen3.uniform_for(seed, request, step))
        else:
            token = plain_qwen3.greedy(row)
            top = torch.topk(row, 2).values
            gap = min(gap, float(top[0] - top[1]))
        out.append(token)
        tokens.append(token)
        if token in eos:
            break
    return (out, gap) if margin else out


@pytest.fixture(scope="module", params=["tiny_a", "tiny_c"])
def case(request, tmp_path_factory):
    return tiny_folder(tmp_path_factory, request.param, seed=3)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_matches_the_plain_implementation(case, dtype):
    from mini_llm_runtime_b200 import LLM
    folder, config, weights = case
    prompts = [random_tokens(config, n, 7 + n) for n in (5, 17, 31)]
    llm = LLM(folder, dtype=dtype, max_model_len=128, max_requests=4, num_pages=32, page_size=4,
              max_batch_tokens=16, prefill_chunk=8)
    results = llm.generate(prompts, max_tokens=8, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert result.finish_reason == "length" and result.prompt_tokens == len(prompt) and len(result.token_ids) == 8
        if dtype == "float32":
            assert result.token_ids == plain_generate(config, weights, prompt, 8)
        else:   # two logits closer than the rounding of bfloat16 may change places; nothing else may
            assert_greedy_tokens(config, weights, prompt, result.token_ids, dtype, f"prompt of {len(prompt)}")
    # Mixed steps happened: decoded tokens beside prompt portions.
    assert any(b["prefill"] and b["decode"] for b in llm.engine.batch_log)
    assert llm.model.cache.free_pages(0) == 32


def test_temperature_sampling_is_reproducible_and_independent_of_batching(case):
    from mini_llm_runtime_b200 import LLM, SamplingParams
    folder, config, weights = case
    prompts = [random_tokens(config, n, 70 + n) for n in (1, 9, 40, 77)]
    params = [SamplingParams(max_tokens=12, temperature=0.7, seed=7, ignore_eos=True) for _ in prompts]
    together = LLM(folder, dtype="float32", max_model_len=128, max_requests=4, num_pages=64, page_size=8,
                   max_batch_tokens=32, prefill_chunk=16).generate(prompts, params=params)
    alone_llm = LLM(folder, dtype="float32", max_model_len=128, max_requests=1, num_pages=16, page_size=8,
                    max_batch_tokens=256, prefill_chunk=128)
    for i, (prompt, result) in enumerate(zip(prompts, together)):
        want = plain_generate(config, weights, prompt, 12, temperature=0.7, seed=7, request=i)
        assert result.token_ids == want, f"request {i}"
    # The same request alone (another engine, request id 0 there) with its id's draws:
    # batching does not enter the draw, only (seed, request, step) does.
    again = alone_llm.generate([prompts[0]], params=[params[0]])
    assert again[0].token_ids == together[0].token_ids
    assert len({tuple(r.token_ids) for r in together}) > 1


def test_end_of_sequence_stops_generation(case):
    from mini_llm_runtime_b200 import LLM
    folder, config, weights = case
    prompt = random_tokens(config, 12, 5)
    free_run = plain_generate(config, weights, prompt, 6)
    eos = free_run[2]
    cfg = dict(config, eos_token_id=eos)
    import tempfile, shutil
    with tempfile.TemporaryDirectory() as tmp:
        shutil.copy(os.path.join(folder, "model.safetensors"), tmp)
        json.dump(cfg, open(os.path.join(tmp, "config.json"), "w"))
        llm = LLM(tmp, dtype="float32", max_model_len=64, max_requests=2, num_pages=8)
        stopped = llm.generate([prompt], max_tokens=6)[0]
        assert stopped.finish_reason == "stop" and stopped.token_ids == free_run[:free_run.index(eos) + 1]
        ignored = llm.generate([prompt], max_tokens=6, ignore_eos=True)[0]
        assert ignored.finish_reason == "length" and ignored.token_ids == free_run


def test_running_ahead_changes_nothing_but_the_timing(case):
    """Several requests decode together and end at different times, some at an
    end-of-sequence id (which the engine only learns after the next step is launched),
    some at their token limit; greedy and with a temperature."""
    from mini_llm_runtime_b200 import LLM, SamplingParams
    folder, config, weights = case
    prompts = [random_tokens(config, n, 90 + n) for n in (6, 11, 3, 20)]
    free_runs = [plain_generate(config, weights, p, 14) for p in prompts]
    eos = [free_runs[0][5], free_runs[1][9]]            # request 0 stops at its 6th token or earlier, request 1 at its 10th
    cfg = dict(config, eos_token_id=eos)
    import tempfile, shutil
    with tempfile.TemporaryDirectory() as tmp:
        shutil.copy(os.path.join(folder, "model.safetensors"), tmp)
        json.dump(cfg, open(os.path.join(tmp, "config.json"), "w"))
        outs = {}
        for ahead in (False, True):
            llm = LLM(tmp, dtype="float32", max_model_len=64, max_requests=4, num_pages=32, page_size=8,
                      max_batch_tokens=64, prefill_chunk=32, run_ahead=ahead)
            params = [SamplingParams(max_tokens=14), SamplingParams(max_tokens=14), SamplingParams(max_tokens=9),
                      SamplingParams(max_tokens=14, temperature=0.8, seed=5)]
            outs[ahead] = llm.generate(prompts, params=params)
            assert (llm.engine.steps_ahead > 0) == ahead
            assert llm.model.cache.free_pages(0) == 32 and llm.model.cache.free_slots() == 4
            llm.model.check_status()
        for a, b in zip(outs[False], outs[True]):
            assert a.token_ids == b.token_ids and a.finish_reason == b.finish_reason
        stops = [r.finish_reason for r in outs[True]]
        assert stops[0] == "stop" and stops[2] == "length" and len(outs[True][2].token_ids) == 9
        for run, result in zip(free_runs[:3], outs[True][:3]):
            assert result.token_ids == run[:len(result.token_ids)]


def test_small_pool_makes_requests_wait_and_pages_are_used_again(case):
    from mini_llm_runtime_b200 import LLM
    folder, config, weights = case
    prompts = [random_tokens(config, 20 + i, 30 + i) for i in range(5)]
    # 8 pages of 8 tokens; a request needs ceil((24+6)/8) = 4: two live at a time.
    llm = LLM(folder, dtype="float32", max_model_len=64, max_requests=4, num_pages=8, page_size=8,
              max_batch_tokens=16, prefill_chunk=8)
    results = llm.generate(prompts, max_tokens=6, ignore_eos=True)
    for prompt, result in zip(prompts, results):
        assert result.token_ids == plain_generate(config, weights, prompt, 6)
    assert all(llm.model.cache.free_pages(g) == 8 for g in range(len(llm.model.cache.groups)))


def test_command_line(case, tmp_path):
    folder, config, weights = case
    prompt = random_tokens(config, 9, 1)
    run = lambda *extra: subprocess.run([sys.executable, os.path.join(ROOT, "bin", "mini-llm"), "--model", folder,
                                         "--prompt-ids", ",".join(map(str, prompt)), *extra],
                                        capture_output=True, text=True)
    done = run("--tokens", "5", "--dtype", "float32", "--ignore-eos", "--context", "64", "--chunk", "4")
    assert done.returncode == 0, done.stderr
    report = json.loads(done.stdout)
    assert report["token_ids"] == plain_generate(config, weights, prompt, 5)
    assert report["prompt_tokens"] == 9 and report["completion_tokens"] == 5 and report["finish_reason"] == "length"
    assert report["used_kv_pages_before_release"] >= 1 and report["used_kv_pages_after_release"] == 0
    assert report["steps"] == 3 + 4          # 9 prompt tokens in portions of 4, then 4 decode steps
    bad = run("--tokens", "0")
    assert bad.returncode == 1 and "out-of-range integer: --tokens" in bad.stderr
    bad = run("--context", "16", "--tokens", "32")
    assert bad.returncode == 1 and "exceed the context budget" in bad.stderr
