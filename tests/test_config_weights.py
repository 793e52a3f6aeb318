"""Configuration, registry, safetensors and loader errors (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

import plain_qwen3
import tiny_models
from mini_llm_runtime_b200 import models as _models  # noqa: F401
from mini_llm_runtime_b200.config.base import ConfigError, Run
from mini_llm_runtime_b200.config.registry import config_from_dict, config_from_dir, known_architectures, plan_for
from mini_llm_runtime_b200.engine.structure import expected_weights
from mini_llm_runtime_b200.weights.loader import WeightMismatch, load_checkpoint
from mini_llm_runtime_b200.weights.random_init import write_random_model
from mini_llm_runtime_b200.weights.safetensors_io import SafetensorsFile, WeightFileError, write_safetensors


@pytest.mark.parametrize("name", list(tiny_models.ALL))
def test_config_reads_every_size(name):
    raw = tiny_models.get(name)
    cfg = config_from_dict(raw)
    assert cfg.hidden_size == raw["hidden_size"] and cfg.num_hidden_layers == raw["num_hidden_layers"]
    assert cfg.num_attention_heads == raw["num_attention_heads"] and cfg.num_key_value_heads == raw["num_key_value_heads"]
    assert cfg.head_dim == raw["head_dim"] and cfg.intermediate_size == raw["intermediate_size"]
    assert cfg.vocab_size == raw["vocab_size"] and cfg.rms_norm_eps == raw["rms_norm_eps"]
    assert cfg.rope_theta == raw["rope_theta"] and cfg.tie_word_embeddings == raw["tie_word_embeddings"]
    assert list(cfg.layer_windows) == plain_qwen3.layer_windows(raw)
    assert config_from_dict(cfg.to_dict()) == cfg


def test_head_dim_defaults_to_width_over_heads():
    raw = tiny_models.get("tiny_a")
    del raw["head_dim"]
    assert config_from_dict(raw).head_dim == 16
    raw["hidden_size"] = 66
    with pytest.raises(ConfigError, match="not divisible"):
        config_from_dict(raw)


def test_layer_types_list_wins():
    raw = tiny_models.get("tiny_c")
    raw["layer_types"] = ["sliding_attention", "full_attention", "full_attention", "sliding_attention"]
    assert config_from_dict(raw).layer_windows == (40, None, None, 40)


@pytest.mark.parametrize("change, match", [
    ({"architectures": ["LlamaForCausalLM"]}, "unknown architecture"),
    ({"architectures": []}, "architectures"),
    ({"hidden_size": None}, "lacks required key 'hidden_size'"),
    ({"rms_norm_eps": None}, "rms_norm_eps"),
    ({"rope_theta": None}, "rope_theta"),
    ({"num_hidden_layers": 0}, "outside"),
    ({"vocab_size": 2_000_000}, "outside"),
    ({"num_key_value_heads": 3}, "not a multiple"),
    ({"head_dim": 15}, "even"),
    ({"rms_norm_eps": 0.0}, "finite and positive"),
    ({"rope_theta": float("inf")}, "finite and positive"),
    ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope scaling"),
    ({"attention_bias": True}, "attention_bias"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"eos_token_id": 999}, "outside the vocabulary"),
])
def test_config_errors(change, match):
    raw = tiny_models.get("tiny_a")
    for k, v in change.items():
        if v is None:
            raw.pop(k)
        else:
            raw[k] = v
    with pytest.raises(ConfigError, match=match):
        config_from_dict(raw)


def test_registry_lists_known_names():
    assert "Qwen3ForCausalLM" in known_architectures()
    with pytest.raises(ConfigError, match="Qwen3ForCausalLM"):
        config_from_dict({"architectures": ["Nope"]})


def test_plan_is_data():
    cfg = config_from_dict(tiny_models.get("tiny_c"))
    plan = plan_for(cfg)
    assert [r.layer for r in plan.schedule] == [0, 1, 2, 3] and all(r.kv_from is None for r in plan.schedule)
    assert [l.mixer.params["window"] for l in plan.layers] == [None, 40, 40, 40]
    assert plan.layers[0].mixer.params["head_dim"] == 48 and plan.layers[0].feed_forward.params["intermediate_size"] == 176
    import dataclasses
    bad = dataclasses.replace(plan, schedule=(Run(0), Run(1, kv_from=3)))
    with pytest.raises(ConfigError, match="not an earlier run"):
        bad.validate()


def test_expected_weights_match_the_architecture():
    for name in tiny_models.ALL:
        raw = tiny_models.get(name)
        specs = expected_weights(plan_for(config_from_dict(raw)))
        assert {k: tuple(v.shape) for k, v in specs.items()} == plain_qwen3.tensor_names(raw)
        assert ("lm_head.weight" in specs) == (not raw["tie_word_embeddings"])


def test_safetensors_round_trip(tmp_path):
    tensors = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.randn(7), "c": torch.arange(6, dtype=torch.int64).view(2, 3),
               "d": torch.randn(2, 2).to(torch.float16)}
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, tensors, {"k": "v"})
    f = SafetensorsFile(path)
    assert sorted(f.names()) == ["a", "b", "c", "d"] and f.metadata == {"k": "v"}
    for n, t in tensors.items():
        assert f.dtype(n) == t.dtype and torch.equal(f.tensor(n), t)
    # The same bytes are what the widely used container format defines.
    from safetensors import safe_open
    with safe_open(path, "pt") as g:
        for n, t in tensors.items():
            assert torch.equal(g.get_tensor(n), t)


def test_safetensors_damage(tmp_path):
    path = str(tmp_path / "x.safetensors")
    write_safetensors(path, {"a": torch.zeros(4, 4)})
    blob = open(path, "rb").read()
    open(path, "wb").write(blob[:-8])
    with pytest.raises(WeightFileError, match="does not fit"):
        SafetensorsFile(path)
    open(path, "wb").write(b"\x05")
    with pytest.raises(WeightFileError, match="shorter"):
        SafetensorsFile(path)
    with pytest.raises(WeightFileError, match="neither"):
        load_checkpoint(str(tmp_path / "nowhere"), {})


def _folder(tmp_path, raw, weights):
    os.makedirs(tmp_path, exist_ok=True)
    json.dump(raw, open(os.path.join(tmp_path, "config.json"), "w"))
    write_safetensors(os.path.join(tmp_path, "model.safetensors"), weights)
    return str(tmp_path)


def test_loader_lists_every_disagreement_at_once(tmp_path):
    raw = tiny_models.get("tiny_b")
    weights = plain_qwen3.random_weights(raw, 0)
    del weights["model.layers.1.mlp.up_proj.weight"]
    del weights["lm_head.weight"]
    weights["model.layers.9.extra.weight"] = torch.zeros(2)
    weights["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(16, dtype=torch.bfloat16)
    weights["model.layers.2.self_attn.k_proj.weight"] = torch.zeros(96, 95, dtype=torch.bfloat16)
    folder = _folder(tmp_path, raw, weights)
    specs = expected_weights(plan_for(config_from_dir(folder)))
    with pytest.raises(WeightMismatch) as e:
        load_checkpoint(folder, specs)
    err = e.value
    assert err.missing == ["lm_head.weight", "model.layers.1.mlp.up_proj.weight"]
    assert err.unexpected == ["model.layers.9.extra.weight"]
    assert [w[0] for w in err.wrong] == ["model.layers.0.self_attn.q_norm.weight", "model.layers.2.self_attn.k_proj.weight"]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "is [16], expected [32]"):
        assert needle in text


def test_loader_keeps_stored_precision(tmp_path):
    raw = tiny_models.get("tiny_a")
    weights = plain_qwen3.random_weights(raw, 0)
    weights["model.norm.weight"] = weights["model.norm.weight"].float()
    folder = _folder(tmp_path, raw, weights)
    specs = expected_weights(plan_for(config_from_dir(folder)))
    loaded = load_checkpoint(folder, specs)
    assert loaded["model.norm.weight"].dtype is torch.float32
    assert loaded["model.embed_tokens.weight"].dtype is torch.bfloat16
    assert torch.equal(loaded["model.layers.1.mlp.down_proj.weight"], weights["model.layers.1.mlp.down_proj.weight"])


def test_tied_head_stored_beside_the_embedding_is_accepted(tmp_path):
    """The reference reads `output.weight` when the file has it and the embedding otherwise
    (src/minillm/qwen3_model.cpp:60-61): a tied checkpoint that stores both copies is the same
    model.  A second copy that differs from the embedding is refused, and so is any other
    extra tensor."""
    raw = tiny_models.get("tiny_a")
    weights = plain_qwen3.random_weights(raw, 0)
    weights["lm_head.weight"] = weights["model.embed_tokens.weight"].clone()
    folder = _folder(tmp_path / "same", raw, weights)
    plan = plan_for(config_from_dir(folder))
    loaded = load_checkpoint(folder, expected_weights(plan), plan.redundant_tensors)
    assert "lm_head.weight" not in loaded and "model.embed_tokens.weight" in loaded
    with pytest.raises(WeightMismatch, match="unexpected .1.: lm_head.weight"):
        load_checkpoint(folder, expected_weights(plan))          # without the plan's word for it, it is unexpected
    weights["lm_head.weight"][3, 5] += 1.0
    folder = _folder(tmp_path / "differs", raw, weights)
    with pytest.raises(WeightFileError, match="the two differ"):
        load_checkpoint(folder, expected_weights(plan), plan.redundant_tensors)
    weights["model.extra.weight"] = torch.zeros(2, 2)
    folder = _folder(tmp_path / "extra", raw, weights)
    with pytest.raises(WeightMismatch, match="unexpected .1.: model.extra.weight"):
        load_checkpoint(folder, expected_weights(plan), plan.redundant_tensors)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    raw = tiny_models.get("tiny_c")
    write_random_model(str(tmp_path / "m"), raw, seed=5)
    write_random_model(str(tmp_path / "n"), raw, seed=5)
    write_random_model(str(tmp_path / "o"), raw, seed=6)
    cfg = config_from_dir(str(tmp_path / "m"))
    specs = expected_weights(plan_for(cfg))
    a, b, c = (load_checkpoint(str(tmp_path / d), specs) for d in "mno")
    assert all(torch.equal(a[k], b[k]) for k in a) and not torch.equal(a["lm_head.weight"], c["lm_head.weight"])
    assert a["lm_head.weight"].dtype is torch.bfloat16
    assert abs(a["lm_head.weight"].float().std() - 0.02) < 2e-3
    norm = a["model.layers.0.input_layernorm.weight"].float()
    assert abs(norm.mean() - 1.0) < 0.01 and 0.003 < norm.std() < 0.03
    # The plain implementation runs on what was written.
    logits = plain_qwen3.forward(raw, a, [1, 2, 3])
    assert logits.shape == (3, raw["vocab_size"]) and torch.isfinite(logits).all()


def test_bench_refuses_several_gpus_and_has_no_reference_arm():
    """The contract of bench.py that needs no GPU: one line and exit code 2 for N > 1; the
    reference arm says in one JSON line why it cannot run and exits 0."""
    import json
    import subprocess
    import sys
    bench = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    many = subprocess.run([sys.executable, bench, "--gpus", "2"], capture_output=True, text=True)
    assert many.returncode == 2 and len(many.stdout.strip().splitlines()) == 1
    reference = subprocess.run([sys.executable, bench, "--impl", "reference"], capture_output=True, text=True)
    line = json.loads(reference.stdout.strip())
    assert reference.returncode == 0 and line["impl"] == "reference" and line["unavailable"]


def test_gate_and_up_rows_interleave_in_blocks_of_128():
    """The operand of the gated product: 128 gate rows, their 128 "up" rows, and so on, the
    last block padded with zero rows; the plain formula applied block by block gives the
    feed-forward's activation back (a CPU restatement of what the kernels read)."""
    from mini_llm_runtime_b200.ops.functions import GATE_BLOCK, interleave_gate_up
    inter, width = 300, 24
    g = torch.Generator().manual_seed(5)
    gate, up = torch.randn(inter, width, generator=g), torch.randn(inter, width, generator=g)
    stacked = interleave_gate_up(gate, up)
    blocks = -(-inter // GATE_BLOCK)
    assert stacked.shape == (2 * blocks * GATE_BLOCK, width)
    x = torch.randn(7, width, generator=g)
    product = (x @ stacked.T).view(7, blocks, 2, GATE_BLOCK)
    silu = lambda t: t / (1 + torch.exp(-t))
    act = silu(product[:, :, 0]) * product[:, :, 1]
    act = act.reshape(7, blocks * GATE_BLOCK)
    want = silu(x @ gate.T) * (x @ up.T)
    assert torch.allclose(act[:, :inter], want, atol=1e-5) and (act[:, inter:] == 0).all()


def test_split_counts_fill_whole_rounds_of_blocks():
    from mini_llm_runtime_b200.ops.functions import k_splits_for
    for rows, K in ((4096, 4096), (24576, 4096), (4096, 12288), (151936, 4096), (1024, 1024), (128, 64)):
        splits = k_splits_for(rows, K, 148)
        units = -(-rows // 128) * splits
        assert 1 <= splits <= 16 and (splits == 1 or -(-K // 64) // splits >= 4)
        if rows * K >= 4096 * 4096:
            assert units / (148 * -(-units // 148)) >= 0.85, (rows, K, splits)


def test_inspect_describes_a_folder_without_a_gpu(tmp_path, capsys):
    """`mini-llm --model DIR --inspect` (the reference's flag, apps/mini_main.cpp:54-71): the
    container, the architecture and its dimensions, and whether the tensors are the expected
    ones; `--output` writes the same report to a file."""
    from mini_llm_runtime_b200 import cli
    folder = str(tmp_path / "m")
    write_random_model(folder, tiny_models.get("tiny_c"), seed=1)
    report_file = str(tmp_path / "report.json")
    assert cli.main(["--model", folder, "--inspect", "--output", report_file]) == 0
    report = json.loads(capsys.readouterr().out)
    assert report == json.load(open(report_file))
    assert report["architecture"] == "Qwen3ForCausalLM" and report["layers"] == 4 and report["runs"] == 4
    assert report["dimensions"]["head_dim"] == 48 and report["dimensions"]["vocab_size"] == 515
    assert report["missing_tensors"] == [] and report["unexpected_tensors"] == []
    assert report["windows"] == ["40", "None"] and report["tensors"] > 10
    assert report["bytes"] == os.path.getsize(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------- the portable generator
def test_portable_generator_is_a_function_of_seed_name_and_index():
    from mini_llm_runtime_b200.weights import portable_random as pr
    a = pr.normal_float32(2, "model.layers.0.mlp.up_proj.weight", 50_000, 0.02)
    assert np.array_equal(a, pr.normal_float32(2, "model.layers.0.mlp.up_proj.weight", 50_000, 0.02, chunk=777))
    assert np.array_equal(a[:100], pr.normal_float32(2, "model.layers.0.mlp.up_proj.weight", 100, 0.02))   # a prefix of itself
    assert not np.array_equal(a, pr.normal_float32(3, "model.layers.0.mlp.up_proj.weight", 50_000, 0.02))
    assert not np.array_equal(a, pr.normal_float32(2, "model.layers.1.mlp.up_proj.weight", 50_000, 0.02))
    assert abs(a.mean()) < 4 * 0.02 / 50_000 ** 0.5 and abs(a.std() - 0.02) < 3e-4
    one = pr.normal_float32(2, "model.norm.weight", 50_000, 0.01, one_plus=True)
    assert abs(one.mean() - 1.0) < 3e-4 and abs(one.std() - 0.01) < 2e-4
    # Pinned values: the device kernel and any other restatement have to give these bits.
    first = pr.normal_float32(0, "w", 4, 1.0).view(np.uint32).tolist()
    assert first == [0xBE134923, 0xBF845A2A, 0xBFCEE0F8, 0xBD1A3326], [hex(v) for v in first]


def test_series_of_the_generator_agree_with_the_library():
    from mini_llm_runtime_b200.weights import portable_random as pr
    u = np.random.default_rng(0).random(200_000)
    u[:4] = [2.0 ** -53, 1.0, 0.5, 0.7071067811865476]
    assert np.abs(pr._ln(u) - np.log(u)).max() < 1e-14
    t = np.random.default_rng(1).random(200_000)
    t[:5] = [0.0, 0.125, 0.25, 0.5, 1.0 - 2.0 ** -53]
    assert np.abs(pr._cos_turns(t) - np.cos(2 * np.pi * t)).max() < 2e-15


@pytest.mark.gpu
def test_device_generator_gives_the_host_generator_bits():
    """numpy on the host and the kernel on the device make the same tensors: every tensor of
    tiny B in both stored precisions, and one matrix of the 8B sizes (12288 x 4096)."""
    from mini_llm_runtime_b200.weights.random_init import random_tensor, random_tensors
    from mini_llm_runtime_b200.weights.loader import WeightSpec
    specs = expected_weights(plan_for(config_from_dict(tiny_models.get("tiny_b"))))
    for dtype in (torch.bfloat16, torch.float32):
        host = random_tensors(specs, 1, dtype, "cpu")
        device = random_tensors(specs, 1, dtype, "cuda:0")
        for name in specs:
            assert torch.equal(host[name], device[name].cpu()), (name, dtype)
    spec = WeightSpec("model.layers.0.mlp.gate_proj.weight", (12288, 4096))
    host = random_tensor(spec.name, spec, 2, torch.bfloat16, "cpu")
    device = random_tensor(spec.name, spec, 2, torch.bfloat16, "cuda:0")
    assert torch.equal(host, device.cpu())
    spec = WeightSpec("model.layers.3.self_attn.o_proj.weight", (1024, 2048))
    assert torch.equal(random_tensor(spec.name, spec, 3, torch.float32, "cpu"),
                       random_tensor(spec.name, spec, 3, torch.float32, "cuda:0").cpu())


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_non_finite_weights_are_refused_by_name(tmp_path, dtype):
    """The reference refuses a checkpoint with a NaN or an infinity while it decodes it
    (src/minillm/cuda/storage.cpp:314-321); here the check runs on the device after the upload and
    the error names every such tensor."""
    from mini_llm_runtime_b200.engine.loading import load_model
    from mini_llm_runtime_b200.engine.runtime import NonFiniteWeights
    raw = tiny_models.get("tiny_b")
    weights = plain_qwen3.random_weights(raw, 0)
    load_model(_folder(tmp_path / "good", raw, weights), dtype)
    weights["model.layers.1.mlp.down_proj.weight"][5, 7] = float("inf")
    weights["model.layers.2.self_attn.k_norm.weight"][3] = float("nan")
    with pytest.raises(NonFiniteWeights) as info:
        load_model(_folder(tmp_path / "bad", raw, weights), dtype)
    assert "(2): model.layers.1.mlp.down_proj.weight, model.layers.2.self_attn.k_norm.weight" in str(info.value)


def test_a_head_size_no_kernel_takes_is_refused_when_the_model_is_planned():
    """The configuration accepts sizes up to a million (src/minillm/qwen3_model.cpp:13-19); the attention kernels of
    this engine end at 256 per head, and say so before any weight is read."""
    from mini_llm_runtime_b200.engine.structure import expected_weights as expected
    raw = dict(tiny_models.get("tiny_a"), head_dim=272)
    with pytest.raises(ConfigError, match="head size 272"):
        expected(plan_for(config_from_dict(raw)))
