"""Can the model-level comparisons fail?  A request's block table is changed for one step,
on valid memory that the request owns, and the comparison with the plain implementation has
to notice, in float32 and in bfloat16.

Attention does not care in which order it meets (key, value) pairs, so two pages that a row
reads whole may change places without any effect (that, too, is checked).  A wrong page
shows where membership matters: at the edge of a sliding window, and at the page a request
is still filling.  Nothing here leaves the pool: the ids that are swapped are the request's
own, no kernel sees an index it must refuse, nothing faults.
"""
import pytest
import torch

import plain_qwen3
from helpers import assert_close, engine_model, random_tokens, tiny_folder

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def case(tmp_path_factory):
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_d", seed=13)     # layer 1 reads a window of 150 keys
    tokens = random_tokens(config, 200, 17)
    return folder, config, tokens, plain_qwen3.forward(config, weights, tokens)


def run(folder, dtype, tokens, first, swap, zero_pool=False):
    """`first` tokens in one step, the rest in a second step whose table has the blocks
    `swap` = (i, j) exchanged in every cache group; logits of the second step."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    model = engine_model(folder, dtype, num_pages=32, page_size=16)
    if zero_pool:
        for r in model.runs:
            r.context.cache.zero_()
    slot = model.open_request()
    model.step([StepEntry(slot, tokens[:first], [])])

    def exchange(group, slots, table):
        i, j = swap
        assert table[0, i] >= 0 and table[0, j] >= 0, "both blocks must be pages the request owns"
        table[0, i], table[0, j] = int(table[0, j]), int(table[0, i])

    model.table_hook = exchange if swap else None
    rest = len(tokens) - first
    logits = model.step([StepEntry(slot, tokens[first:], list(range(rest)))]).float().cpu()
    model.table_hook = None
    model.check_status()
    return logits


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wrong_page_is_noticed(case, dtype):
    folder, config, tokens, want = case
    # The step as it should be.
    assert_close(run(folder, dtype, tokens, 166, None), want[166:], dtype, "no mutation")
    # Two pages every row of the step reads whole, in both layers' sight: no effect beyond rounding.
    assert_close(run(folder, dtype, tokens, 166, (4, 6)), want[166:], dtype, "two pages that are read whole")
    # Block 1 (positions 16..31) lies before the window of the rows from position 181 on and partly
    # before that of the others, block 5 inside everyone's: the windowed layer now reads keys
    # 16..31 in the place of keys 80..95.
    with pytest.raises(AssertionError, match="differ|are off"):
        assert_close(run(folder, dtype, tokens, 166, (1, 5)), want[166:], dtype, "a page across the window's edge")
    # The page the request is still filling (positions 144..149 of the first step) against a full
    # one: the step writes its new rows into the wrong page and reads six old rows from the other.
    # The pool starts from zeros here, so that the rows never written are finite.
    assert_close(run(folder, dtype, tokens, 150, None, zero_pool=True), want[150:], dtype, "no mutation, zeroed pool")
    with pytest.raises(AssertionError, match="differ|are off"):
        assert_close(run(folder, dtype, tokens, 150, (4, 9), zero_pool=True), want[150:], dtype, "the page being filled")
