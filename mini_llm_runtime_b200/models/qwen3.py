"""Qwen3 dense decoder as a model plan.

The architecture is the one src/minillm/qwen3_model.cpp binds and
src/minillm/runtime.cpp:245-351 runs: per layer a pre-norm block of grouped-query
attention (per-head RMS norm of q and k, half-split rotation, causal) and a
SiLU-gated feed-forward; a final RMS norm; an output head that is its own matrix
or the embedding table.  This module only turns a `Qwen3Config` into data; the
parts it names live in `parts/`.
"""
from __future__ import annotations

import math

from ..config.base import LayerSpec, ModelPlan, PartSpec, Run
from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    norm = lambda name: PartSpec("rmsnorm", {"width": cfg.hidden_size, "eps": cfg.rms_norm_eps},
                                 {"weight": name})
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        mixer = PartSpec(
            "attention",
            {"hidden_size": cfg.hidden_size, "num_heads": cfg.num_attention_heads,
             "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
             "scale": 1.0 / math.sqrt(cfg.head_dim), "window": cfg.layer_windows[i],
             "qk_norm_eps": cfg.rms_norm_eps, "position": "rope"},
            {"q": p + "self_attn.q_proj.weight", "k": p + "self_attn.k_proj.weight",
             "v": p + "self_attn.v_proj.weight", "o": p + "self_attn.o_proj.weight",
             "q_norm": p + "self_attn.q_norm.weight", "k_norm": p + "self_attn.k_norm.weight"})
        ff = PartSpec(
            "swiglu", {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size},
            {"gate": p + "mlp.gate_proj.weight", "up": p + "mlp.up_proj.weight",
             "down": p + "mlp.down_proj.weight"})
        layers.append(LayerSpec(
            block="pre_norm", mixer=mixer, feed_forward=ff,
            norms={"pre_mixer": norm(p + "input_layernorm.weight"),
                   "pre_feed_forward": norm(p + "post_attention_layernorm.weight")}))
    embed_name = "model.embed_tokens.weight"
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "width": cfg.hidden_size},
                           {"weight": embed_name}),
        positions={"rope": PartSpec("rope", {"theta": cfg.rope_theta, "rotary_dim": cfg.head_dim,
                                             "max_positions": cfg.max_position_embeddings})},
        layers=tuple(layers),
        schedule=tuple(Run(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm("model.norm.weight"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "width": cfg.hidden_size},
                         {"weight": embed_name if cfg.tie_word_embeddings else "lm_head.weight"}),
        eos_token_ids=cfg.eos_token_ids,
        # The reference takes `output.weight` when the file has it and the embedding otherwise
        # (src/minillm/qwen3_model.cpp:60-61); a tied checkpoint that stores both is the same model.
        redundant_tensors=(("lm_head.weight", embed_name),) if cfg.tie_word_embeddings else (),
    )


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_plan)
