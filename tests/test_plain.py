"""The plain implementation checked against itself (no GPU): properties that hold
for the architecture whatever the weights are."""
import math

import pytest
import torch

import plain_qwen3
import plain_qwen3 as P
import tiny_models


@pytest.fixture(scope="module")
def models():
    return {n: (tiny_models.get(n), P.random_weights(tiny_models.get(n), i)) for i, n in enumerate(tiny_models.ALL)}


def test_float32_and_float64_agree(models):
    for name, (cfg, w) in models.items():
        tokens = torch.randint(0, cfg["vocab_size"], (40,), generator=torch.Generator().manual_seed(3)).tolist()
        a = P.forward(cfg, w, tokens, torch.float32)
        b = P.forward(cfg, w, tokens, torch.float64)
        assert (a.double() - b).abs().max() < 2e-5, name


def test_causality(models):
    cfg, w = models["tiny_b"]
    tokens = list(range(10, 40))
    changed = tokens[:20] + [t + 1 for t in tokens[20:]]
    a, b = P.forward(cfg, w, tokens), P.forward(cfg, w, changed)
    assert torch.equal(a[:20], b[:20]) and not torch.allclose(a[20:], b[20:])
    assert torch.allclose(P.forward(cfg, w, tokens[:7]), a[:7], atol=1e-6)


def test_rms_norm_and_rope_formulas():
    x = torch.tensor([[3.0, -4.0, 0.0, 0.0]])
    w = torch.tensor([1.0, 2.0, 1.0, 1.0])
    out = P.rms_norm(x, w, 1e-6)
    scale = 1.0 / math.sqrt((9 + 16) / 4 + 1e-6)
    assert torch.allclose(out, torch.tensor([[3 * scale, -8 * scale, 0.0, 0.0]]))
    cos, sin = P.rope_table([0, 1, 5], 8, 10000.0, torch.float32)
    assert torch.equal(cos[0], torch.ones(4)) and torch.equal(sin[0], torch.zeros(4))
    assert torch.allclose(cos[2], torch.cos(5.0 * 10000.0 ** (-2 * torch.arange(4.0) / 8)))
    # Rotation keeps the norm, and q.k depends only on the distance between positions.
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 8, generator=g), torch.randn(1, 1, 8, generator=g)
    c, s = P.rope_table(range(30), 8, 10000.0, torch.float32)
    rot = lambda v, p: P.apply_rope(v, c[p:p + 1], s[p:p + 1])
    assert torch.allclose(rot(q, 7).norm(), q.norm(), atol=1e-5)
    d1 = (rot(q, 12) * rot(k, 9)).sum()
    d2 = (rot(q, 23) * rot(k, 20)).sum()
    assert torch.allclose(d1, d2, atol=1e-4)
    # Half-split pairing: element j rotates with element j + D/2.
    e0 = torch.zeros(1, 1, 8); e0[0, 0, 0] = 1.0
    r = rot(e0, 3)[0, 0]
    assert r[0] == c[3, 0] and r[4] == s[3, 0] and r[1:4].abs().sum() == 0


def test_attention_reads_the_right_kv_head_and_window():
    T, Hq, Hkv, D = 12, 6, 2, 4
    g = torch.Generator().manual_seed(1)
    q, k, v = torch.randn(T, Hq, D, generator=g), torch.randn(T, Hkv, D, generator=g), torch.randn(T, Hkv, D, generator=g)
    out = P.causal_attention(q, k, v)
    # Dense formulation of the same thing.
    for h in range(Hq):
        kv = h // 3
        s = (q[:, h] @ k[:, kv].T) / math.sqrt(D)
        s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        assert torch.allclose(out[:, h], torch.softmax(s, -1) @ v[:, kv], atol=1e-6)
    win = P.causal_attention(q, k, v, window=3)
    assert torch.allclose(win[:3], out[:3], atol=1e-6) and not torch.allclose(win[3:], out[3:])
    # A window of 1 returns the row's own value.
    one = P.causal_attention(q, k, v, window=1)
    assert torch.allclose(one[:, 4], v[:, 1], atol=1e-6)
    # The first position attends to itself only.
    assert torch.allclose(out[0, 0], v[0, 0])


def test_window_changes_only_far_context(models):
    cfg, w = models["tiny_c"]
    tokens = torch.randint(0, cfg["vocab_size"], (70,), generator=torch.Generator().manual_seed(4)).tolist()
    full_cfg = dict(cfg, use_sliding_window=False)
    a, b = P.forward(cfg, w, tokens), P.forward(full_cfg, w, tokens)
    assert torch.allclose(a[:40], b[:40], atol=1e-6)      # within the window nothing is cut
    assert (a[45:] - b[45:]).abs().max() > 1e-5


def test_tied_head_and_schedule(models):
    cfg, w = models["tiny_a"]
    h = P.forward(cfg, w, [1, 2, 3], return_hidden=True)
    logits = P.forward(cfg, w, [1, 2, 3])
    f = P.rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    assert torch.allclose(logits, f @ w["model.embed_tokens.weight"].float().T)
    twice = P.forward(cfg, w, [1, 2, 3, 4], schedule=[(0, None), (1, None), (0, None)])
    shared = P.forward(cfg, w, [1, 2, 3, 4], schedule=[(0, None), (1, 0)])
    plain = P.forward(cfg, w, [1, 2, 3, 4])
    assert not torch.allclose(twice, plain) and not torch.allclose(shared, plain)


def test_sampling_definitions():
    row = torch.tensor([0.5, 2.0, 2.0, -1.0])
    assert P.greedy(row) == 1
    us = [P.uniform_for(7, r, s) for r in range(20) for s in range(20)]
    assert all(0 <= u < 1 for u in us) and len(set(us)) == 400 and 0.4 < sum(us) / 400 < 0.6
    assert P.uniform_for(7, 3, 5) == P.uniform_for(7, 3, 5) != P.uniform_for(8, 3, 5)
    cdf = P.temperature_cdf(row, 1.0)
    p = torch.softmax(row.double(), 0)
    assert torch.allclose(cdf, torch.cumsum(p, 0), atol=1e-6)
    assert P.sample_temperature(row, 1.0, 0.0) == 0 and P.sample_temperature(row, 1.0, 0.999999) == 3
    assert P.sample_temperature(row, 1.0, float(p[0]) + 1e-6) == 1
    assert P.sample_temperature(row, 0.0, 0.3) == 1
    # The engine's restatement of the uniform draw is the same function.
    from mini_llm_runtime_b200.sampling.sampler import uniform_for
    assert all(uniform_for(s, r, t) == P.uniform_for(s, r, t) for s in (0, 7, 2**40) for r in (0, 5) for t in (0, 9))


def test_dense_restatement_equals_the_loop():
    """`plain_dense.forward_rows` (the oracle at real sizes) against `plain_qwen3.forward`, with
    and without a window, for all rows and for chosen rows."""
    import plain_dense
    for name, seed in (("tiny_b", 3), ("tiny_c", 4)):
        config = tiny_models.get(name)
        weights = plain_qwen3.random_weights(config, seed)
        tokens = torch.randint(0, config["vocab_size"], (90,), generator=torch.Generator().manual_seed(seed)).tolist()
        loop = plain_qwen3.forward(config, weights, tokens, dtype=torch.float64)
        dense = plain_dense.forward_rows(config, weights, tokens)
        assert torch.allclose(loop, dense, atol=1e-9, rtol=0)
        assert torch.allclose(plain_dense.forward_rows(config, weights, tokens, rows=[0, 41, 89]), dense[[0, 41, 89]], atol=1e-12, rtol=0)
        small_blocks = plain_dense.dense_attention(*(torch.randn(70, h, 16, dtype=torch.float64) for h in (6, 2, 2)), window=9, block=16)
        assert torch.isfinite(small_blocks).all()
