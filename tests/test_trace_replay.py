"""Trace replay through `bin/trace_run`: the same requests whole, with the last 32
tokens one by one, in portions of changing size, and mixed with other requests in a
pool so small that pages are used again; in float32 and bfloat16; every logits row
against the plain implementation, and the float32 modes against each other bit for
bit."""
import pytest
import torch

import plain_qwen3
import trace_tools as T
from helpers import assert_close, random_tokens, tiny_folder

pytestmark = pytest.mark.gpu

LENGTHS = {"tiny_a": [100, 37, 128, 65, 80, 51], "tiny_b": [150, 33, 97, 256, 64, 70], "tiny_c": [200, 41, 130, 75, 300, 66],
           "tiny_d": [330, 70, 200, 129, 262, 90]}
MODES = {"whole": T.whole, "last32": T.last_32_one_by_one, "portions": T.portions,
         "mixed": lambda r: T.mixed(r, seed=11)}


@pytest.fixture(scope="module", params=list(LENGTHS))
def case(request, tmp_path_factory):
    name = request.param
    folder, config, weights = tiny_folder(tmp_path_factory, name, seed=len(name))
    requests = {f"r{i}": random_tokens(config, n, 50 + i) for i, n in enumerate(LENGTHS[name])}
    want = {k: plain_qwen3.forward(config, weights, t) for k, t in requests.items()}
    return name, folder, config, requests, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_modes_match_the_plain_implementation(case, dtype, tmp_path):
    name, folder, config, requests, want = case
    results = {}
    for mode, make in MODES.items():
        trace = make(requests)
        if mode == "mixed":
            # Pages must be used again: the pool is smaller than all requests together.
            assert T.max_live_tokens(trace) < sum(T.round64(len(t)) for t in requests.values())
            assert max(len(s["entries"]) for s in trace) >= 3
            assert any(len(e["tokens"]) > 1 for s in trace for e in s["entries"] if len(s["entries"]) > 1)
        logits = T.run_trace(folder, dtype, trace, str(tmp_path / mode), config["vocab_size"])
        results[mode] = logits
        for k, tokens in requests.items():
            assert_close(T.stack(logits, k, len(tokens)), want[k], dtype, f"{name} {mode} request {k}")
    if dtype == "float32":
        # The 32-bit kernels fix each output's order of summation, so cutting and batching
        # change nothing at all.
        for mode in ("last32", "portions", "mixed"):
            for key, row in results["whole"].items():
                assert torch.equal(row, results[mode][key]), f"{name} {mode} differs from whole at {key}"


def test_replay_with_pages_of_64_tokens(case, tmp_path):
    """The same mixed trace in a pool of 64-token pages (one copy per key tile in the
    attention kernels instead of four)."""
    name, folder, config, requests, want = case
    if name != "tiny_d":
        pytest.skip("one configuration is enough here")
    trace = T.mixed(requests, seed=12)
    logits = T.run_trace(folder, "bfloat16", trace, str(tmp_path / "p64"), config["vocab_size"], page_size=64)
    for k, tokens in requests.items():
        assert_close(T.stack(logits, k, len(tokens)), want[k], "bfloat16", f"{name} pages of 64, request {k}")


def test_steps_without_wanted_logits_and_requests_left_out(case, tmp_path):
    name, folder, config, requests, want = case
    a, b = requests["r0"], requests["r1"]
    trace = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:10], "want": []}], "end": []},
        {"step": 1, "entries": [{"id": "b", "tokens": b[:5], "want": [4]}], "end": []},
        {"step": 2, "entries": [{"id": "a", "tokens": a[10:12], "want": [1]}, {"id": "b", "tokens": b[5:6]}], "end": ["b"]},
        {"step": 3, "entries": [], "end": []},
        {"step": 4, "entries": [{"id": "a", "tokens": a[12:13], "want": [0]}], "end": ["a"]},
    ]
    logits = T.run_trace(folder, "float32", trace, str(tmp_path / "o"), config["vocab_size"], max_tokens=128)
    assert sorted(logits) == [("a", 11), ("a", 12), ("b", 4)]
    assert_close(logits[("a", 11)][None], want["r0"][11:12], "float32")
    assert_close(logits[("a", 12)][None], want["r0"][12:13], "float32")
    assert_close(logits[("b", 4)][None], want["r1"][4:5], "float32")
