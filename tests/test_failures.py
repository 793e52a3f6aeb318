"""What a failed step leaves behind.  Every failure here is made on the host: a launch
wrapper that raises instead of launching, a part whose forward raises, a status word set
by the test, a step function replaced by a fake.  No kernel is given a bad address and
nothing faults or hangs the GPU; the reference tests its runtime the same way, with wrapped
CUDA calls that fail after real completion and a fake runner under its engine
(tests/cuda_runtime_tests.cpp:15-49, tests/core_tests.cpp:500-594).

The rules under test (src/minillm/cuda/runtime.cpp:216-253, src/minillm/cuda/page_table.cpp:91-96):
  * a step refused before device work (a bad batch, a pool that cannot hold it) changes
    nothing and the model stays usable;
  * a step that fails after device work began rolls back its pages, lengths and the
    fixed-size state of its requests, and poisons the model: no further step or request;
  * a status word a kernel set poisons the model before a token of that step is handed out.
"""
import dataclasses

import pytest
import torch

import plain_qwen3 as P
from helpers import engine_model, random_tokens, tiny_folder

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folder_b(tmp_path_factory):
    return tiny_folder(tmp_path_factory, "tiny_b", seed=5)


def ledger(model, slots=(0, 1)):
    cache = model.cache
    return ([cache.free_pages(g) for g in range(len(cache.groups))], cache.free_slots(), [cache.length(s) for s in slots])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nth", [0, 3, 11])
def test_a_launch_that_fails_mid_step_rolls_back_and_poisons(folder_b, dtype, nth):
    from mini_llm_runtime_b200.engine.model import Poisoned, StepEntry
    from mini_llm_runtime_b200.ops import native
    folder, config, weights = folder_b
    tokens = random_tokens(config, 40, 1)
    model = engine_model(folder, dtype, num_pages=16, page_size=8)
    a, b = model.open_request(), model.open_request()
    first = model.step([StepEntry(a, tokens[:10], [9]), StepEntry(b, tokens[:3], [])]).clone()
    before = ledger(model)
    native.fail_after(nth)
    try:
        with pytest.raises(native.KernelError, match="injected failure"):
            model.step([StepEntry(a, tokens[10:30], [19]), StepEntry(b, [tokens[3]], [0])])
    finally:
        native.fail_after(None)
    assert ledger(model) == before, "pages, slots or lengths of the failed step were kept"
    assert model.poisoned is not None and "injected failure" in model.poisoned
    with pytest.raises(Poisoned):
        model.step([StepEntry(a, tokens[10:12], [])])
    with pytest.raises(Poisoned):
        model.open_request()
    model.close_request(a)                         # giving back is still allowed
    model.close_request(b)
    assert model.cache.free_pages(0) == 16 and model.cache.free_slots() == 4
    # The device itself is fine: nothing faulted, the first step's logits can still be read.
    assert torch.isfinite(first).all() and int(model.status.item()) == 0


def test_a_step_refused_before_device_work_changes_nothing(folder_b):
    from mini_llm_runtime_b200.cache.manager import OutOfPages
    from mini_llm_runtime_b200.engine.model import StepEntry, StepError
    folder, config, weights = folder_b
    tokens = random_tokens(config, 60, 2)
    model = engine_model(folder, "float32", num_pages=4, page_size=8)
    a = model.open_request()
    model.step([StepEntry(a, tokens[:20], [])])
    before = ledger(model, [a])
    with pytest.raises(OutOfPages):
        model.step([StepEntry(a, tokens[20:60], [])])            # 60 tokens need 8 pages, the pool has 4
    with pytest.raises(StepError):
        model.step([StepEntry(a, [config["vocab_size"]], [0])])
    with pytest.raises(StepError):
        model.step([StepEntry(a, tokens[20:22], [2])])
    assert ledger(model, [a]) == before and model.poisoned is None
    want = P.forward(config, weights, tokens[:28])
    got = model.step([StepEntry(a, tokens[20:28], [7])]).cpu()
    assert torch.allclose(got, want[27:28], atol=2e-4, rtol=2e-4)


def test_fixed_size_state_is_inside_the_transaction(tmp_path_factory):
    """A mixer that keeps a running sum per request, then a feed-forward that raises: the sum
    the mixer had already advanced in the failed step is put back."""
    from mini_llm_runtime_b200.config.base import LayerSpec, PartSpec, Run
    from mini_llm_runtime_b200.config.registry import config_from_dir, plan_for, register_part
    from mini_llm_runtime_b200.engine.model import CacheConfig, Model, Poisoned, StepEntry
    from mini_llm_runtime_b200.engine.runtime import Runtime
    from mini_llm_runtime_b200.parts.base import FeedForward, Mixer, StateNeed

    class RunningSum(Mixer):
        def state_need(self):
            return StateNeed((self.spec.params["width"],), torch.float32)

        def forward(self, x, step, run):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for seg in step.segments:
                sums = run.state[seg.slot] + torch.cumsum(x[seg.row:seg.row + seg.count].float(), 0)
                run.state[seg.slot] = sums[-1]
                out[seg.row:seg.row + seg.count] = sums * 0.01
            return out

    class FailsOnDemand(FeedForward):
        fail = False

        def forward(self, x, step):
            if FailsOnDemand.fail:
                raise RuntimeError("the feed-forward failed")
            return torch.zeros(x.shape, dtype=torch.float32, device=x.device)

    register_part("mixer", "test_running_sum", RunningSum)
    register_part("feed_forward", "test_fails_on_demand", FailsOnDemand)
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_a", seed=9)
    base = plan_for(config_from_dir(folder))
    toy = LayerSpec(block="pre_norm", mixer=PartSpec("test_running_sum", {"width": config["hidden_size"]}),
                    feed_forward=PartSpec("test_fails_on_demand"), norms=base.layers[1].norms)
    plan = dataclasses.replace(base, layers=(base.layers[0], toy), schedule=(Run(0), Run(1)))
    model = Model(plan, Runtime(torch.float32))
    model.bind({n: weights[n] for n in model.expected_weights()})
    model.allocate_cache(CacheConfig(page_size=4, num_pages=32, max_requests=2))
    tokens = random_tokens(config, 30, 3)
    a, b = model.open_request(), model.open_request()
    model.step([StepEntry(a, tokens[:7], []), StepEntry(b, tokens[:2], [])])
    state = model.runs[1].context.state
    kept, before = state.clone(), ledger(model)
    assert kept.abs().sum() > 0
    FailsOnDemand.fail = True
    try:
        with pytest.raises(RuntimeError, match="the feed-forward failed"):
            model.step([StepEntry(a, tokens[7:19], [11]), StepEntry(b, [tokens[2]], [0])])
    finally:
        FailsOnDemand.fail = False
    assert torch.equal(state, kept), "the failed step left the requests' state advanced"
    assert ledger(model) == before
    with pytest.raises(Poisoned):
        model.step([StepEntry(a, tokens[7:9], [])])


def test_a_status_word_poisons_the_model(folder_b):
    from mini_llm_runtime_b200.engine.model import DeviceFault, Poisoned, StepEntry
    folder, config, weights = folder_b
    model = engine_model(folder, "float32", num_pages=8, page_size=8)
    a = model.open_request()
    model.step([StepEntry(a, [1, 2, 3], [2])])
    model.check_status()
    model.status.fill_(2)                  # what a kernel does when it meets a page id outside the pool
    with pytest.raises(DeviceFault, match="status 2"):
        model.check_status()
    with pytest.raises(Poisoned):
        model.step([StepEntry(a, [4], [0])])


@pytest.mark.parametrize("run_ahead", [False, True])
def test_engine_hands_out_nothing_after_a_reported_fault(folder_b, run_ahead):
    """The status word is read back with a step's ids; when a kernel has set it, no request of
    that step advances, the call raises, and the engine refuses to go on."""
    from mini_llm_runtime_b200 import LLM
    from mini_llm_runtime_b200.engine.model import DeviceFault, Poisoned
    folder, config, weights = folder_b
    llm = LLM(folder, dtype="float32", max_model_len=64, max_requests=2, num_pages=16, run_ahead=run_ahead)
    engine = llm.engine
    ids = [engine.submit(random_tokens(config, 6, i)) for i in range(2)]
    engine.step()
    engine.step()
    generated = [list(r.generated) for r in engine.scheduler.active]
    assert all(len(g) >= 1 for g in generated)
    llm.model.status.fill_(4)
    with pytest.raises(DeviceFault):
        engine.step()
        engine.step()          # with run-ahead the fault is read one call later
    assert all(len(r.generated) <= len(g) + 1 for r, g in zip(engine.scheduler.active, generated))
    handed_out = [list(r.generated) for r in engine.scheduler.active]
    with pytest.raises(Poisoned):
        engine.step()
    assert [list(r.generated) for r in engine.scheduler.active] == handed_out and len(ids) == 2


def test_engine_over_a_step_function_that_fails(folder_b):
    """A fake step function under the engine: one that raises, one that returns too few rows.
    The engine hands out no token of such a step and refuses to go on; credits and slots of
    the requests can still be given back."""
    from mini_llm_runtime_b200 import LLM
    from mini_llm_runtime_b200.engine.model import Poisoned
    folder, config, weights = folder_b
    for kind in ("raises", "short"):
        llm = LLM(folder, dtype="float32", max_model_len=64, max_requests=3, num_pages=24)
        engine, model = llm.engine, llm.model
        for i in range(3):
            engine.submit(random_tokens(config, 5 + i, i))
        engine.step()
        real_step = model.step

        def fake(entries, device_tokens=None, kind=kind):
            if kind == "raises":
                raise RuntimeError("the step function failed")
            return real_step(entries, device_tokens)[:1]

        model.step = fake
        reserved = list(engine.scheduler.reserved)
        tokens_before = [list(r.generated) for r in engine.scheduler.active]
        with pytest.raises(RuntimeError, match="step function"):
            for _ in range(3):
                engine.step()
        assert [list(r.generated)[:len(t)] for r, t in zip(engine.scheduler.active, tokens_before)] == tokens_before
        if kind == "short":
            assert model.poisoned is not None
            with pytest.raises(Poisoned):
                engine.step()
        assert engine.scheduler.reserved == reserved          # nothing was released behind the requests' backs
        for r in list(engine.scheduler.active):
            model.close_request(r.slot)
            engine.scheduler.release(r)
        assert engine.scheduler.reserved == [0] * len(reserved) and model.cache.free_slots() == 3
        assert model.cache.free_pages(0) == 24
