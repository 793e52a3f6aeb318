"""Each part alone against the plain implementation's function for it, the run order
as data (a layer run twice, a run that reads another run's cache), and a toy mixer
with state of its own that is defined here, registered, built and stepped without
any change to the package; likewise a toy feed-forward with routing and a toy position
encoding.  The toy parts use torch operations: they show the interfaces, not kernels."""
import dataclasses
import math

import pytest
import torch

import plain_qwen3 as P
import tiny_models
from helpers import assert_close, random_tokens, tiny_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def runtime(dtype):
    from mini_llm_runtime_b200.engine.runtime import Runtime
    return Runtime(dtype, DEV)


def fake_step(rt, segments, page_size=16, tables=None):
    """A StepContext for parts that are called outside a model."""
    from mini_llm_runtime_b200.parts.base import Segment, StepContext
    segs, pos, seg_of, info, row = [], [], [], [], 0
    for i, (start, count) in enumerate(segments):
        segs.append(Segment(i, start, count, row))
        pos += list(range(start, start + count))
        seg_of += [i] * count
        info.append([row, count, start, i])
        row += count
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return StepContext(rt=rt, num_rows=row, segments=segs, token_ids=t([0] * row), positions=t(pos),
                       segment_of_row=t(seg_of), segment_info=t(info), slots=t(list(range(len(segs)))),
                       tables=tables or {}, page_size=page_size, status=torch.zeros(1, dtype=torch.int32, device=DEV),
                       max_count=max(c for _, c in segments), max_context=max(s + c for s, c in segments),
                       all_single=all(c == 1 for _, c in segments))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.parts.norm import RmsNorm
    rt = runtime(dtype)
    part = RmsNorm(PartSpec("rmsnorm", {"width": 80, "eps": 3e-6}, {"weight": "w"}))
    assert [(s.name, s.shape, s.role) for s in part.weight_specs()] == [("w", (80,), "vector")]
    w = (1 + 0.1 * torch.randn(80)).to(torch.bfloat16)
    part.bind({"w": w}, rt)
    h, delta = torch.randn(5, 80), torch.randn(5, 80)
    hd = h.to(DEV)
    out = part.forward(hd, delta.to(DEV), fake_step(rt, [(0, 5)]))
    assert out.dtype is dtype and torch.equal(hd.cpu(), h + delta)
    want = P.rms_norm(h + delta, w.float(), 3e-6)
    assert torch.allclose(out.float().cpu(), want, atol=1e-5 if dtype is torch.float32 else 2e-2, rtol=1e-2)


def test_rope_part_table_is_the_reference_formula():
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.parts.rotary import Rope
    part = Rope(PartSpec("rope", {"theta": 1e6, "rotary_dim": 48, "max_positions": 300}))
    part.bind({}, runtime(torch.float32))
    table = part.rotation_table().cpu()
    cos, sin = P.rope_table(range(300), 48, 1e6, torch.float32)
    assert table.shape == (300, 48)
    assert torch.allclose(table[:, :24], cos, atol=2e-7) and torch.allclose(table[:, 24:], sin, atol=2e-7)
    assert part.weight_specs() == []


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.parts.mlp import SwiGLU
    rt = runtime(dtype)
    H, I = 80, 176
    part = SwiGLU(PartSpec("swiglu", {"hidden_size": H, "intermediate_size": I}, {"gate": "g", "up": "u", "down": "d"}))
    assert sorted((s.name, s.shape) for s in part.weight_specs()) == [("d", (H, I)), ("g", (I, H)), ("u", (I, H))]
    w = {"g": torch.randn(I, H) * 0.1, "u": torch.randn(I, H) * 0.1, "d": torch.randn(H, I) * 0.1}
    w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    part.bind(w, rt)
    x = torch.randn(7, H).to(torch.bfloat16)
    out = part.forward(x.to(DEV).to(dtype), fake_step(rt, [(0, 7)]))
    assert out.dtype is torch.float32           # a delta for the float32 residual stream
    names = {"p.mlp.gate_proj.weight": w["g"], "p.mlp.up_proj.weight": w["u"], "p.mlp.down_proj.weight": w["d"]}
    want = P.swiglu_mlp(x.float(), names, "p.")
    assert torch.allclose(out.cpu(), want, atol=1e-5 if dtype is torch.float32 else 2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype,head_dim", [(torch.float32, 48), (torch.bfloat16, 48), (torch.bfloat16, 64)])
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_with_its_cache(dtype, head_dim, window):
    """The mixer alone: two requests, one in two portions, against the plain attention."""
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.parts.attention import AttentionMixer
    from mini_llm_runtime_b200.parts.base import CacheNeed, RunContext
    from mini_llm_runtime_b200.parts.rotary import Rope
    rt = runtime(dtype)
    H, Hq, Hkv, D, eps, theta = 40, 6, 2, head_dim, 1e-5, 5e4
    cfg = {"hidden_size": H, "num_attention_heads": Hq, "num_key_value_heads": Hkv, "head_dim": D, "rms_norm_eps": eps}
    part = AttentionMixer(PartSpec("attention", {"hidden_size": H, "num_heads": Hq, "num_kv_heads": Hkv, "head_dim": D,
                                                 "scale": 1 / math.sqrt(D), "window": window, "qk_norm_eps": eps,
                                                 "position": "rope"},
                                   {r: f"p.self_attn.{r}_proj.weight" for r in "qkvo"} |
                                   {"q_norm": "p.self_attn.q_norm.weight", "k_norm": "p.self_attn.k_norm.weight"}))
    assert part.cache_need() == CacheNeed(window, Hkv, D) and part.state_need() is None
    w = {s.name: ((1 + 0.1 * torch.randn(s.shape)) if s.role == "vector" else torch.randn(s.shape) * 0.08).to(torch.bfloat16)
         for s in part.weight_specs()}
    assert len(w) == 6
    part.position = Rope(PartSpec("rope", {"theta": theta, "rotary_dim": D, "max_positions": 64}))
    part.position.bind({}, rt)
    part.bind(w, rt)
    lengths = [23, 11]
    xs = [torch.randn(n, H).to(torch.bfloat16) for n in lengths]
    wants = []
    for x in xs:
        cos, sin = P.rope_table(range(len(x)), D, theta, torch.float32)
        q, k, v = P.attention_projections(x.float(), w, "p.", cfg, cos, sin)
        o = P.causal_attention(q, k, v, window)
        wants.append(o.reshape(len(x), -1) @ w["p.self_attn.o_proj.weight"].float().T)
    page, pages = 4, 12
    cache = torch.full((pages, 2, Hkv, page, D), float("nan"), dtype=dtype, device=DEV)
    table = torch.tensor([[5, 0, 7, 2, 9, 11], [3, 8, 1, -1, -1, -1]], dtype=torch.int32, device=DEV)
    run = RunContext(group=0, cache=cache, write_cache=True)
    outs = [[], []]
    # Step 1: 14 tokens of request 0 beside all of request 1; step 2: the rest of request 0.
    for segments, rows in [([(0, 14), (0, 11)], [xs[0][:14], xs[1]]), ([(14, 9)], [xs[0][14:]])]:
        step = fake_step(rt, segments, page_size=page, tables={0: table[:len(segments)].contiguous()})
        out = part.forward(torch.cat(rows).to(DEV).to(dtype), step, run).cpu()
        assert step.status.item() == 0
        offset = 0
        for i, (_, count) in enumerate(segments):
            outs[i].append(out[offset:offset + count])
            offset += count
    tol = dict(atol=2e-5, rtol=1e-4) if dtype is torch.float32 else dict(atol=3e-2, rtol=3e-2)
    for got, want in zip(outs, wants):
        assert torch.allclose(torch.cat(got), want, **tol)


def test_pre_norm_block_folds_the_residual_adds():
    """The block's output with a pending contribution equals the plain layer on h + pending."""
    from mini_llm_runtime_b200.config.registry import config_from_dict, plan_for
    from mini_llm_runtime_b200.engine.model import CacheConfig, Model, StepEntry
    raw = tiny_models.get("tiny_a")
    raw["num_hidden_layers"] = 1
    weights = P.random_weights(raw, 5)
    rt = runtime(torch.float32)
    model = Model(plan_for(config_from_dict(raw)), rt)
    model.bind(weights)
    model.allocate_cache(CacheConfig(page_size=4, num_pages=8, max_requests=1))
    tokens = [5, 6, 7, 8, 9]
    slot = model.open_request()
    # Run the block by hand on a step the model prepared.
    logits = model.step([StepEntry(slot, tokens, [4])])
    want = P.forward(raw, weights, tokens)
    assert_close(logits.cpu(), want[4:], "float32", "one-layer model")
    block = model.blocks[0]
    assert set(block.norms) == {"pre_mixer", "pre_feed_forward"}
    assert type(block).__name__ == "PreNormBlock" and block.mixer.position is model.positions["rope"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_run_order_is_data(tmp_path_factory, dtype):
    """A plan that runs layer 0 twice and lets a later run read an earlier run's cache."""
    from mini_llm_runtime_b200.config.base import Run
    from mini_llm_runtime_b200.config.registry import config_from_dir, plan_for
    from mini_llm_runtime_b200.engine.model import CacheConfig, Model
    from mini_llm_runtime_b200.weights.loader import load_checkpoint
    from helpers import run_portions, run_whole
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_b", seed=8)
    tokens = random_tokens(config, 90, 3)
    for schedule in ([(0, None), (1, None), (0, None), (2, None)], [(0, None), (1, None), (2, 0), (1, 1)]):
        plan = dataclasses.replace(plan_for(config_from_dir(folder)), schedule=tuple(Run(l, k) for l, k in schedule))
        model = Model(plan, runtime(torch.float32 if dtype == "float32" else torch.bfloat16))
        model.bind(load_checkpoint(folder, model.expected_weights()))
        model.allocate_cache(CacheConfig(page_size=8, num_pages=24, max_requests=2))
        caches = {id(r.context.cache) for r in model.runs}
        assert len(caches) == len([1 for _, k in schedule if k is None])      # a run of its own has a cache of its own
        want = P.forward(config, weights, tokens, schedule=schedule)
        assert_close(run_whole(model, tokens), want, dtype, f"schedule {schedule} whole")
        assert_close(run_portions(model, tokens, [33, 2, 17, 1]), want, dtype, f"schedule {schedule} in portions")


def test_a_toy_mixer_with_state_is_added_from_outside(tmp_path_factory):
    """A mixer that keeps a running sum per request: registered here, built by the
    generic model beside an attention layer, stepped in portions and mixed batches.
    Nothing in the package knows it."""
    from mini_llm_runtime_b200.config.base import LayerSpec, PartSpec, Run
    from mini_llm_runtime_b200.config.registry import config_from_dir, plan_for, register_part
    from mini_llm_runtime_b200.engine.model import CacheConfig, Model, StepEntry
    from mini_llm_runtime_b200.parts.base import Mixer, StateNeed
    from mini_llm_runtime_b200.weights.loader import WeightSpec, load_checkpoint

    class RunningMean(Mixer):
        """delta[t] = W mean(x[0..t]); the state is the sum over the tokens seen so far."""
        def __init__(self, spec):
            super().__init__(spec)
            self.width = spec.params["width"]

        def state_need(self):
            return StateNeed((self.width,), torch.float32)

        def weight_specs(self):
            return [WeightSpec(self.spec.weights["w"], (self.width, self.width))]

        def bind(self, tensors, rt):
            self.w = tensors[self.spec.weights["w"]].to(rt.device).float()

        def forward(self, x, step, run):
            out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            for seg in step.segments:
                rows = x[seg.row:seg.row + seg.count].float()
                sums = run.state[seg.slot] + torch.cumsum(rows, 0)
                run.state[seg.slot] = sums[-1]
                counts = torch.arange(seg.start + 1, seg.start + seg.count + 1, device=x.device)[:, None]
                out[seg.row:seg.row + seg.count] = (sums / counts) @ self.w.T
            return out

    register_part("mixer", "test_running_mean", RunningMean)
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_a", seed=9)
    base = plan_for(config_from_dir(folder))
    H = config["hidden_size"]
    toy_layer = LayerSpec(block="pre_norm", mixer=PartSpec("test_running_mean", {"width": H}, {"w": "toy.w"}),
                          feed_forward=base.layers[1].feed_forward, norms=base.layers[1].norms)
    plan = dataclasses.replace(base, layers=(base.layers[0], toy_layer), schedule=(Run(0), Run(1)))
    toy_w = (torch.randn(H, H, generator=torch.Generator().manual_seed(1)) * 0.05).to(torch.bfloat16)
    model = Model(plan, runtime(torch.float32))
    expected = model.expected_weights()
    assert "toy.w" in expected and "model.layers.1.self_attn.q_proj.weight" not in expected
    tensors = {n: (toy_w if n == "toy.w" else weights[n]) for n in expected}
    model.bind(tensors)
    model.allocate_cache(CacheConfig(page_size=4, num_pages=64, max_requests=3))
    assert model.runs[1].context.state.shape == (3, H) and model.runs[1].context.cache is None
    assert model._native is None                   # a mixer with state: the model is stepped from Python, never from a graph

    def plain(tokens):
        """Layer 0 as the plain implementation has it, layer 1 with the toy mixer."""
        T = len(tokens)
        h = P.embedding(weights["model.embed_tokens.weight"], tokens, torch.float32)
        cos, sin = P.rope_table(range(T), config["head_dim"], config["rope_theta"], torch.float32)
        h, _ = P.decoder_layer(h, weights, 0, config, cos, sin, None)
        p = "model.layers.1."
        n = P.rms_norm(h, weights[p + "input_layernorm.weight"], config["rms_norm_eps"])
        mean = torch.cumsum(n, 0) / torch.arange(1, T + 1)[:, None]
        h = h + mean @ toy_w.float().T
        n2 = P.rms_norm(h, weights[p + "post_attention_layernorm.weight"], config["rms_norm_eps"])
        h = h + P.swiglu_mlp(n2, weights, p)
        return P.final_logits(h, weights, config)

    a, b = random_tokens(config, 40, 1), random_tokens(config, 25, 2)
    want_a, want_b = plain(a), plain(b)
    sa, sb = model.open_request(), model.open_request()
    got_a, got_b = [], []
    # Portions of a beside portions and single tokens of b; b sits a step out.
    plan_steps = [((0, 7), (0, 3)), ((7, 2), None), ((9, 20), (3, 1)), ((29, 1), (4, 1)), ((30, 10), (5, 20))]
    for part_a, part_b in plan_steps:
        entries = [StepEntry(sa, a[part_a[0]:part_a[0] + part_a[1]], list(range(part_a[1])))]
        if part_b:
            entries.append(StepEntry(sb, b[part_b[0]:part_b[0] + part_b[1]], list(range(part_b[1]))))
        logits = model.step(entries).cpu()
        got_a.append(logits[:part_a[1]])
        if part_b:
            got_b.append(logits[part_a[1]:])
    assert_close(torch.cat(got_a), want_a, "float32", "toy model, request a")
    assert_close(torch.cat(got_b), want_b, "float32", "toy model, request b")
    # A slot that is used again starts from an empty state.
    model.close_request(sa)
    sc = model.open_request()
    assert sc == sa
    assert_close(model.step([StepEntry(sc, b, list(range(len(b))))]).cpu(), want_b, "float32", "reused slot")


def test_a_toy_feed_forward_with_routing_is_added_from_outside(tmp_path_factory):
    """Two experts and a router that sends each token to one of them: a FeedForward
    registered here and put into the second layer of an otherwise ordinary model."""
    from mini_llm_runtime_b200.config.base import LayerSpec, PartSpec, Run
    from mini_llm_runtime_b200.config.registry import config_from_dir, plan_for, register_part
    from mini_llm_runtime_b200.engine.model import CacheConfig, Model
    from mini_llm_runtime_b200.parts.base import FeedForward
    from mini_llm_runtime_b200.weights.loader import WeightSpec
    from helpers import run_portions, run_whole

    def routed(x, router, up, down):
        """x [M, W] float32 -> sum over the chosen expert only: p_e * down_e relu(up_e x)."""
        probs = torch.softmax(x @ router.T, dim=-1)
        choice = probs.argmax(-1)
        out = torch.zeros_like(x)
        for e in range(router.shape[0]):
            rows = choice == e
            hidden = torch.relu(x[rows] @ up[e].T)
            out[rows] = probs[rows, e:e + 1] * (hidden @ down[e].T)
        return out

    class TopOneExperts(FeedForward):
        graph_safe = False       # indexing by a mask reads the count of chosen rows back to the host

        def __init__(self, spec):
            super().__init__(spec)
            self.width, self.inter, self.experts = (spec.params[k] for k in ("width", "inter", "experts"))

        def weight_specs(self):
            w = self.spec.weights
            return [WeightSpec(w["router"], (self.experts, self.width)),
                    WeightSpec(w["up"], (self.experts * self.inter, self.width)),
                    WeightSpec(w["down"], (self.experts * self.width, self.inter))]

        def bind(self, tensors, rt):
            w = self.spec.weights
            on = lambda name: tensors[w[name]].to(rt.device).float()
            self.router = on("router")
            self.up = on("up").view(self.experts, self.inter, self.width)
            self.down = on("down").view(self.experts, self.width, self.inter)

        def forward(self, x, step):
            return routed(x.float(), self.router, self.up, self.down)      # a float32 contribution to the stream

    register_part("feed_forward", "test_top_one_experts", TopOneExperts)
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_a", seed=12)
    base = plan_for(config_from_dir(folder))
    H, I, E = config["hidden_size"], 24, 2
    toy = PartSpec("test_top_one_experts", {"width": H, "inter": I, "experts": E},
                   {"router": "toy.router", "up": "toy.up", "down": "toy.down"})
    plan = dataclasses.replace(base, layers=(base.layers[0], dataclasses.replace(base.layers[1], feed_forward=toy)))
    g = torch.Generator().manual_seed(4)
    toy_w = {"toy.router": torch.randn(E, H, generator=g), "toy.up": torch.randn(E * I, H, generator=g) * 0.1,
             "toy.down": torch.randn(E * H, I, generator=g) * 0.1}
    model = Model(plan, runtime(torch.float32))
    expected = model.expected_weights()
    assert "toy.router" in expected and "model.layers.1.mlp.gate_proj.weight" not in expected
    assert "model.layers.0.mlp.gate_proj.weight" in expected and "model.layers.1.self_attn.q_proj.weight" in expected
    model.bind({n: toy_w[n] if n in toy_w else weights[n] for n in expected})
    model.allocate_cache(CacheConfig(page_size=4, num_pages=64, max_requests=2))
    assert model._native is None

    def plain(tokens):
        T = len(tokens)
        h = P.embedding(weights["model.embed_tokens.weight"], tokens, torch.float32)
        cos, sin = P.rope_table(range(T), config["head_dim"], config["rope_theta"], torch.float32)
        h, _ = P.decoder_layer(h, weights, 0, config, cos, sin, None)
        # Layer 1 with its own feed-forward silenced, then the toy one in its place.
        silent = dict(weights)
        silent["model.layers.1.mlp.down_proj.weight"] = torch.zeros_like(weights["model.layers.1.mlp.down_proj.weight"])
        h, _ = P.decoder_layer(h, silent, 1, config, cos, sin, None)
        n = P.rms_norm(h, weights["model.layers.1.post_attention_layernorm.weight"], config["rms_norm_eps"])
        h = h + routed(n, toy_w["toy.router"], toy_w["toy.up"].view(E, I, H), toy_w["toy.down"].view(E, H, I))
        return P.final_logits(h, weights, config)

    tokens = random_tokens(config, 50, 6)
    want = plain(tokens)
    chosen = torch.softmax(P.rms_norm(torch.randn(50, H, generator=g), torch.ones(H), 1e-6) @ toy_w["toy.router"].T, -1).argmax(-1)
    assert 0 < int(chosen.sum()) < 50                      # both experts are in use for inputs of this kind
    assert_close(run_whole(model, tokens), want, "float32", "routed feed-forward, whole")
    assert_close(run_portions(model, tokens, [19, 2, 1, 7]), want, "float32", "routed feed-forward, in portions")


def test_a_toy_position_encoding_is_added_from_outside(tmp_path_factory):
    """Learned absolute positions added to the embedded tokens, and attention that does not
    rotate: a PositionEncoding registered here, named by the plan in place of the rotary one."""
    from mini_llm_runtime_b200.config.base import PartSpec
    from mini_llm_runtime_b200.config.registry import config_from_dir, plan_for, register_part
    from mini_llm_runtime_b200.engine.model import CacheConfig, Model
    from mini_llm_runtime_b200.parts.base import PositionEncoding
    from mini_llm_runtime_b200.weights.loader import WeightSpec
    from helpers import run_portions, run_whole

    class LearnedPositions(PositionEncoding):
        def weight_specs(self):
            return [WeightSpec(self.spec.weights["table"], (self.spec.params["max_positions"], self.spec.params["width"]))]

        def bind(self, tensors, rt):
            self.table = tensors[self.spec.weights["table"]].to(rt.device).float()

        def add_to_embedding(self, h, step):
            h += self.table[step.positions.long()]

    register_part("position", "test_learned_positions", LearnedPositions)
    folder, config, weights = tiny_folder(tmp_path_factory, "tiny_b", seed=13)
    base = plan_for(config_from_dir(folder))
    H, positions = config["hidden_size"], 128
    layers = tuple(dataclasses.replace(l, mixer=dataclasses.replace(l.mixer, params={**l.mixer.params, "position": None}))
                   for l in base.layers)
    plan = dataclasses.replace(base, layers=layers, positions={
        "learned": PartSpec("test_learned_positions", {"max_positions": positions, "width": H}, {"table": "toy.positions"})})
    table = torch.randn(positions, H, generator=torch.Generator().manual_seed(2)) * 0.5
    for dtype in ("float32", "bfloat16"):
        model = Model(plan, runtime(torch.float32 if dtype == "float32" else torch.bfloat16))
        expected = model.expected_weights()
        assert "toy.positions" in expected
        model.bind({n: table if n == "toy.positions" else weights[n] for n in expected})
        model.allocate_cache(CacheConfig(page_size=8, num_pages=32, max_requests=2))
        assert all(b.mixer.position is None for b in model.blocks)

        tokens = random_tokens(config, 70, 9)
        T = len(tokens)
        h = P.embedding(weights["model.embed_tokens.weight"], tokens, torch.float32) + table[:T]
        no_turn = (torch.ones(T, config["head_dim"] // 2), torch.zeros(T, config["head_dim"] // 2))
        for layer in range(config["num_hidden_layers"]):
            h, _ = P.decoder_layer(h, weights, layer, config, *no_turn, None)
        want = P.final_logits(h, weights, config)
        assert_close(run_whole(model, tokens), want, dtype, "learned positions, whole")
        assert_close(run_portions(model, tokens, [33, 1, 2, 20]), want, dtype, "learned positions, in portions")
