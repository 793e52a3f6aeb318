"""Each request alone and whole: the engine's logits at every position against the
plain implementation, in float32 and in bfloat16."""
import pytest
import torch

import plain_qwen3
from helpers import assert_close, engine_model, random_tokens, run_portions, run_whole, tiny_folder

pytestmark = pytest.mark.gpu

CASES = [("tiny_a", 0, 100), ("tiny_b", 1, 150), ("tiny_c", 2, 200), ("tiny_d", 3, 333)]


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


@pytest.mark.parametrize("filler", [float("nan"), 1e30, -7.0])
def test_first_tokens_do_not_depend_on_what_memory_held_before(tmp_path_factory, filler):
    """Every buffer of a fresh model lies in memory that held something else before.  A kernel that reads what the
    kernel before it writes BEFORE that kernel has finished (a load moved above the wait of a programmatic dependent
    launch) sees that old content; the first steps of a small model, where launches follow each other fastest, show it."""
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_d", seed=3)
    tokens = random_tokens(config, 8, 103)
    want = plain_qwen3.forward(config, weights, tokens)
    for trial in range(4):
        held = [torch.empty(1 << 20, dtype=torch.float32, device="cuda:0").fill_(filler) for _ in range(64)]
        del held                                    # the allocator hands these blocks to the model next
        model = engine_model(folder, "bfloat16", num_pages=32)
        for n in (1, 2, 3):
            assert_close(run_whole(model, tokens[:n]), want[:n], "bfloat16", f"trial {trial}, first {n} tokens over memory full of {filler}")
        del model


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_one_by_one(case, dtype):
    folder, config, tokens, want = case
    model = engine_model(folder, dtype, num_pages=32)
    got = run_portions(model, tokens, [len(tokens) - 32, 1])
    assert_close(got, want, dtype, "prompt then 32 single tokens")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_graphs_and_eagerly(case, dtype):
    """Token by token from the first token on, past page edges and graph buckets; the
    graph replay and the plain launches give the same bits."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, tokens, want = case
    outs = {}
    for graphs in (True, False):
        model = engine_model(folder, dtype, num_pages=32)
        model.use_graphs = graphs
        model.graph_bucket_blocks = 2          # new graphs every 32 tokens
        slot = model.open_request()
        rows = [model.step([StepEntry(slot, [t], [0])]).float().cpu() for t in tokens]
        model.check_status()
        outs[graphs] = torch.cat(rows)
        assert bool(model._graphs) == graphs
    assert_close(outs[True], want, dtype, "one token at a time")
    assert torch.equal(outs[True], outs[False])


def test_device_tokens_feed_the_next_step(case):
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, tokens, want = case
    model = engine_model(folder, "float32", num_pages=32)
    slot = model.open_request()
    model.step([StepEntry(slot, tokens[:20], [])])
    for p in range(20, 30):
        ids = torch.tensor([tokens[p]], dtype=torch.int32, device="cuda:0")
        logits = model.step([StepEntry(slot, [0], [0])], device_tokens=ids)
        assert_close(logits.float().cpu(), want[p:p + 1], "float32", f"position {p}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_whole_and_in_large_portions(tmp_path_factory, dtype):
    """2000 tokens: many query tiles and key tiles, waves of attention blocks, over a
    hundred pages, the window of the second layer far behind; in one step, in portions of
    800 (remainders of every kind), and with pages of 64 tokens."""
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_d", seed=21)
    tokens = random_tokens(config, 2000, 77)
    want = plain_qwen3.forward(config, weights, tokens)
    model = engine_model(folder, dtype, num_pages=2 * 128, page_size=16, max_requests=2)
    model.rt.pair_min_tiles = 1      # a tiny model has few tiles: let its gated product take the two-SM kernel all the same
    assert_close(run_whole(model, tokens), want, dtype, "long prompt, whole")
    assert_close(run_portions(model, tokens, [800, 800, 337, 63]), want, dtype, "long prompt, in portions")
    model64 = engine_model(folder, dtype, num_pages=2 * 32, page_size=64, max_requests=2)
    assert_close(run_portions(model64, tokens, [1500, 1, 1, 498]), want, dtype, "long prompt, pages of 64")


def test_every_product_on_the_own_kernel(tmp_path_factory):
    """The mode without the vendor library: prompt portions, decoded tokens and a batch of
    more than 8 rows all go through the package's tcgen05 product."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_d", seed=31)
    tokens = random_tokens(config, 300, 5)
    want = plain_qwen3.forward(config, weights, tokens)
    model = engine_model(folder, "bfloat16", num_pages=64, max_requests=16)
    model.rt.own_products_only()
    assert_close(run_whole(model, tokens), want, "bfloat16", "own products, whole")
    assert_close(run_portions(model, tokens, [200, 70, 1]), want, "bfloat16", "own products, portions and single tokens")
    # Twelve requests decode together (more rows than the default hands to the own kernel).
    slots = [model.open_request() for _ in range(12)]
    model.step([StepEntry(s, tokens[:20 + i], []) for i, s in enumerate(slots)])
    logits = model.step([StepEntry(s, [tokens[20 + i]], [0]) for i, s in enumerate(slots)]).float().cpu()
    model.check_status()
    for i in range(12):
        assert_close(logits[i:i + 1], want[20 + i:21 + i], "bfloat16", f"own products, request {i} of a batch of 12")


@pytest.mark.parametrize("gemv_rows,fuse_rows", [(8, 32), (2, 32), (0, 32), (8, 0)])
def test_few_row_products_on_both_routes(tmp_path_factory, gemv_rows, fuse_rows):
    """Decode steps of up to `Runtime.gemv_rows` rows run on the kernel that norms its own input, gates, adds into the
    stream and prepares the next norm; with 0 the split-K products, the library and the row-wise kernels between
    them take those steps (and with 2, steps of three to eight rows).  One request token by token, and eight
    requests together, on each; the programs name the kernels that were meant.  With `fuse_rotation_rows` the split-KV
    attention kernel makes its own queries, keys and values from the product's raw output in steps of tokens only."""
    from mini_llm_runtime_b200.engine.model import StepEntry
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_d", seed=41)
    tokens = random_tokens(config, 120, 6)
    want = plain_qwen3.forward(config, weights, tokens)
    model = engine_model(folder, "bfloat16", num_pages=96, max_requests=8)
    model.rt.gemv_rows = gemv_rows
    model.rt.fuse_rotation_rows = fuse_rows
    assert_close(run_portions(model, tokens, [60, 1]), want, "bfloat16", "token by token")
    slots = [model.open_request() for _ in range(8)]
    model.step([StepEntry(s, tokens[:30 + i], []) for i, s in enumerate(slots)])
    for step in range(4):
        logits = model.step([StepEntry(s, [tokens[30 + i + step]], [0]) for i, s in enumerate(slots)]).float().cpu()
        for i in range(8):
            assert_close(logits[i:i + 1], want[30 + i + step:31 + i + step], "bfloat16", f"request {i} of eight, step {step}")
    model.step([StepEntry(slots[0], [tokens[34]], [0])])           # (a workspace that grew dropped the programs built before)
    model.check_status()
    programs = model._native.programs
    one_row = next(names for (lo, hi, _, _), names in programs.items() if lo <= 1 <= hi)
    eight_rows = next(names for (lo, hi, _, _), names in programs.items() if lo <= 8 <= hi)
    assert ("mlr_gemv_bf16_prepared" in one_row) == (gemv_rows > 0) and ("mlr_gemv_bf16_prepared" in eight_rows) == (gemv_rows == 8)
    assert ("mlr_rmsnorm" in eight_rows) == (gemv_rows < 8)
    # (where the other route's q/k/v product leaves split-K partial sums, only the row-wise kernel can add them up;
    # at these sizes it goes to the library, so the attention kernel may make its own rows there too)
    if gemv_rows > 0:
        assert ("mlr_attention_decode_fresh_bf16" in one_row) == (fuse_rows > 0)


def test_thirty_two_query_heads_per_kv_head_decode_from_graphs(tmp_path_factory):
    """More than 16 query heads per kv head: single tokens then take the flash kernel with a tile list instead
    of the split-KV kernel.  The list travels in the step's metadata, so such steps are captured and replayed
    like any other decode step."""
    import tiny_models
    from helpers import write_model_folder
    from mini_llm_runtime_b200.engine.model import StepEntry
    config = dict(tiny_models.get("tiny_a"), num_attention_heads=32, num_key_value_heads=1, head_dim=16, hidden_size=64)
    weights = plain_qwen3.random_weights(config, 17)
    folder = str(tmp_path_factory.mktemp("group32"))
    write_model_folder(folder, config, weights)
    tokens = random_tokens(config, 60, 3)
    want = plain_qwen3.forward(config, weights, tokens)
    for dtype in ("bfloat16", "float32"):
        model = engine_model(folder, dtype, num_pages=16)
        slot = model.open_request()
        rows = [model.step([StepEntry(slot, tokens[:20], list(range(20)))]).float().cpu()]
        rows += [model.step([StepEntry(slot, [t], [0])]).float().cpu() for t in tokens[20:]]
        model.check_status()
        assert model._graphs
        assert_close(torch.cat(rows), want, dtype, f"32 query heads per kv head, {dtype}")
