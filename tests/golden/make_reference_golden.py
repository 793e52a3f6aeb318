#!/usr/bin/env python3
"""Makes the golden logits under tests/golden/ by running the REFERENCE's own CPU forward
pass (lilong555/mini-llm-runtime, src/minillm/runtime.cpp) on tiny random models.

    python tests/golden/make_reference_golden.py [/path/to/mini-llm-runtime]

The reference's sources are compiled unchanged from its tree with g++ -std=c++20; only
`GgufModel` and `Tokenizer`, which need llama.cpp, are replaced by the stand-ins in
anchor_shim.cpp.  For each tiny configuration a seeded random model (the same tensors
`tests/plain_qwen3.random_weights` makes) is written to a flat file, one token sequence
is fed whole and again in portions of 7 with logits at every position, and the result is
saved as `<name>.reference_logits.f32` beside the tokens in `<name>.json`.
`tests/test_golden.py` compares the plain implementation with these files.

Two properties of the reference bound how close the comparison can be: its key/value
cache is float16 (src/minillm/paged_kv.cpp:85-98), and it has no sliding window, so only
configurations without a window are anchored.
"""
import json
import os
import struct
import subprocess
import sys
import tempfile

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import plain_qwen3  # noqa: E402
import tiny_models  # noqa: E402

SOURCES = ["src/minillm/kernels.cpp", "src/minillm/paged_kv.cpp", "src/minillm/parallel.cpp",
           "src/minillm/qwen3_model.cpp", "src/minillm/runtime.cpp"]
GGUF_NAMES = {"model.embed_tokens.weight": "token_embd.weight", "model.norm.weight": "output_norm.weight",
              "lm_head.weight": "output.weight"}
LAYER_NAMES = {"input_layernorm.weight": "attn_norm.weight", "self_attn.q_proj.weight": "attn_q.weight",
               "self_attn.k_proj.weight": "attn_k.weight", "self_attn.v_proj.weight": "attn_v.weight",
               "self_attn.q_norm.weight": "attn_q_norm.weight", "self_attn.k_norm.weight": "attn_k_norm.weight",
               "self_attn.o_proj.weight": "attn_output.weight", "post_attention_layernorm.weight": "ffn_norm.weight",
               "mlp.gate_proj.weight": "ffn_gate.weight", "mlp.up_proj.weight": "ffn_up.weight",
               "mlp.down_proj.weight": "ffn_down.weight"}
CASES = {"tiny_a": (0, 41), "tiny_b": (1, 60)}      # name -> (weight seed, sequence length)


def gguf_name(name: str) -> str:
    if name in GGUF_NAMES:
        return GGUF_NAMES[name]
    _, _, index, rest = name.split(".", 3)
    return f"blk.{index}.{LAYER_NAMES[rest]}"


def put_string(f, s: str):
    raw = s.encode()
    f.write(struct.pack("<i", len(raw)) + raw)


def write_model(path: str, cfg: dict, weights: dict):
    meta = [("general.architecture", 2, "qwen3"),
            ("qwen3.embedding_length", 0, cfg["hidden_size"]), ("qwen3.block_count", 0, cfg["num_hidden_layers"]),
            ("qwen3.attention.head_count", 0, cfg["num_attention_heads"]),
            ("qwen3.attention.head_count_kv", 0, cfg["num_key_value_heads"]),
            ("qwen3.attention.key_length", 0, cfg["head_dim"]), ("qwen3.attention.value_length", 0, cfg["head_dim"]),
            ("qwen3.feed_forward_length", 0, cfg["intermediate_size"]),
            ("qwen3.context_length", 0, cfg["max_position_embeddings"]),
            ("qwen3.attention.layer_norm_rms_epsilon", 1, cfg["rms_norm_eps"]),
            ("qwen3.rope.freq_base", 1, cfg["rope_theta"])]
    with open(path, "wb") as f:
        f.write(struct.pack("<i", len(meta)))
        for key, kind, value in meta:
            put_string(f, key)
            f.write(struct.pack("<i", kind))
            if kind == 0:
                f.write(struct.pack("<q", value))
            elif kind == 1:
                f.write(struct.pack("<f", value))
            else:
                put_string(f, value)
        f.write(struct.pack("<i", len(weights)))
        for name, t in weights.items():
            put_string(f, gguf_name(name))
            rows, columns = (1, t.shape[0]) if t.dim() == 1 else t.shape
            f.write(struct.pack("<ii", rows, columns))
            f.write(t.float().contiguous().numpy().astype("<f4").tobytes())


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_reference_golden.py <checkout of lilong555/mini-llm-runtime>")
    reference = sys.argv[1]
    with tempfile.TemporaryDirectory() as tmp:
        binary = os.path.join(tmp, "anchor")
        command = ["g++", "-std=c++20", "-O1", "-pthread", "-I", os.path.join(reference, "include"),
                   os.path.join(HERE, "anchor_shim.cpp"), *[os.path.join(reference, s) for s in SOURCES], "-o", binary]
        subprocess.run(command, check=True)
        for name, (seed, length) in CASES.items():
            cfg = tiny_models.get(name)
            weights = plain_qwen3.random_weights(cfg, seed)
            model = os.path.join(tmp, name + ".bin")
            write_model(model, cfg, weights)
            g = torch.Generator().manual_seed(1000 + seed)
            tokens = torch.randint(0, cfg["vocab_size"], (length,), generator=g).tolist()
            outputs = {}
            for label, portion in (("whole", length), ("portions_of_7", 7)):
                out = os.path.join(tmp, f"{name}.{label}.f32")
                subprocess.run([binary, model, "128", "4", out, str(portion), *map(str, tokens)], check=True)
                outputs[label] = np.fromfile(out, dtype="<f4").reshape(length, cfg["vocab_size"])
            # The reference's own chunking invariance (tests/model_tests.cpp:339-345).
            assert np.abs(outputs["whole"] - outputs["portions_of_7"]).max() < 1e-5
            outputs["whole"].astype("<f4").tofile(os.path.join(HERE, f"{name}.reference_logits.f32"))
            with open(os.path.join(HERE, f"{name}.json"), "w") as f:
                json.dump({"config": name, "weight_seed": seed, "tokens": tokens, "vocab": cfg["vocab_size"],
                           "made_by": "tests/golden/make_reference_golden.py from src/minillm/runtime.cpp"}, f)
            print(name, outputs["whole"].shape, "max |logit|", float(np.abs(outputs["whole"]).max()))


if __name__ == "__main__":
    main()
