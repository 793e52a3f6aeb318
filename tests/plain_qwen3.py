"""Plain, slow Qwen3-dense forward pass: the oracle every engine test compares with.

Whole sequences, no cache, no batching, one function per part, CPU tensors only.
It shares no code with the package under test: it has its own tensor-name table,
its own rope table and its own attention loop.  Every function restates a formula
of lilong555/mini-llm-runtime's CPU runtime and cites where that formula stands
(paths are relative to that project's root).

Two things go beyond the reference, which has neither: a sliding window (keys
older than `window` positions are not read) and a layer schedule (a list that may
run a layer twice or let a run read another run's keys and values).  They are
defined here so that the engine's generality can be tested; with `window=None`
and the identity schedule the functions are exactly the reference's.

All arithmetic is done in `dtype` (float32 by default; float64 gives a higher
precision truth for tolerance calibration).  The softmax denominator is always
summed in float64, as the reference does.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch


# --------------------------------------------------------------------------- names
def tensor_names(cfg: dict) -> Dict[str, tuple]:
    """Checkpoint tensor names and `[rows, columns]` shapes of a Qwen3 dense model.

    The reference binds each tensor by name with an exact shape check
    (src/minillm/qwen3_model.cpp:42-53, :57-80); rows = outputs, columns = inputs,
    `y = x @ W.T` (include/minillm/cuda/matrix.h:35).  The names used here are the
    safetensors names of the same tensors.
    """
    H, L = cfg["hidden_size"], cfg["num_hidden_layers"]
    Hq, Hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim") or H // Hq
    I, V = cfg["intermediate_size"], cfg["vocab_size"]
    names = {"model.embed_tokens.weight": (V, H), "model.norm.weight": (H,)}
    if not cfg.get("tie_word_embeddings", False):
        names["lm_head.weight"] = (V, H)
    for i in range(L):
        p = f"model.layers.{i}."
        names[p + "input_layernorm.weight"] = (H,)
        names[p + "self_attn.q_proj.weight"] = (Hq * D, H)
        names[p + "self_attn.k_proj.weight"] = (Hkv * D, H)
        names[p + "self_attn.v_proj.weight"] = (Hkv * D, H)
        names[p + "self_attn.q_norm.weight"] = (D,)
        names[p + "self_attn.k_norm.weight"] = (D,)
        names[p + "self_attn.o_proj.weight"] = (H, Hq * D)
        names[p + "post_attention_layernorm.weight"] = (H,)
        names[p + "mlp.gate_proj.weight"] = (I, H)
        names[p + "mlp.up_proj.weight"] = (I, H)
        names[p + "mlp.down_proj.weight"] = (H, I)
    return names


def random_weights(cfg: dict, seed: int, store_dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Seeded random tensors for a config: matrices ~ N(0, 0.02), norm weights
    1 + N(0, 0.01), rounded once to `store_dtype` so that every path sees the same
    values.  (The reference's own fixture fills weights with a counter pattern,
    tests/qwen3_fixture.h:48-54; a normal distribution is used here instead.)
    """
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_names(cfg).items():
        if len(shape) == 1:
            t = 1.0 + 0.01 * torch.randn(shape, generator=g, dtype=torch.float32)
        else:
            t = 0.02 * torch.randn(shape, generator=g, dtype=torch.float32)
        out[name] = t.to(store_dtype)
    return out


def layer_windows(cfg: dict) -> List[Optional[int]]:
    """Per layer: None for full causal attention or the window length.

    The reference reads every key `t <= position` (src/minillm/runtime.cpp:287,294),
    i.e. `use_sliding_window = false`.  With `use_sliding_window = true` the config
    keys `sliding_window` and `max_window_layers` say that layers with index
    `>= max_window_layers` read only the last `sliding_window` keys; a `layer_types`
    list, when present, names each layer's kind directly.
    """
    L = cfg["num_hidden_layers"]
    if not cfg.get("use_sliding_window", False) or cfg.get("sliding_window") is None:
        return [None] * L
    if cfg.get("layer_types"):
        return [cfg["sliding_window"] if t == "sliding_attention" else None for t in cfg["layer_types"]]
    first = cfg.get("max_window_layers", L)
    return [cfg["sliding_window"] if i >= first else None for i in range(L)]


# --------------------------------------------------------------------------- parts
def embedding(table: torch.Tensor, tokens: Sequence[int], dtype) -> torch.Tensor:
    """`h[r, :] = E[token[r], :]`, a row copy without scaling (src/minillm/runtime.cpp:224-228)."""
    return table.to(dtype)[torch.as_tensor(list(tokens), dtype=torch.long)]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """`(x * (1 / sqrt(mean(x^2) + eps))) * w`: scale first, then the weight
    (src/minillm/kernels.cpp:209-216).  The mean runs over the last dimension."""
    dtype = x.dtype
    scale = 1.0 / torch.sqrt((x * x).sum(-1, keepdim=True) / x.shape[-1] + torch.tensor(eps, dtype=dtype))
    return (x * scale) * weight.to(dtype)


def rope_table(positions: Sequence[int], head_dim: int, theta: float, dtype):
    """cos/sin of `angle = float(pos) * theta^(-2j/D)`, j in [0, D/2).

    The reference computes frequency, angle, cosine and sine in float
    (src/minillm/runtime.cpp:231-241); the same is done here in float32 whatever
    `dtype` is, then the table is widened to `dtype`."""
    half = head_dim // 2
    # `std::pow(float, float)` is the C library's powf; numpy's float32 power calls the same
    # function, while torch's vectorised pow may differ from it in the last bit, which the
    # position then multiplies.
    j = np.arange(half, dtype=np.float32)
    exponent = (np.float32(-2.0) * j / np.float32(head_dim)).astype(np.float32)
    freq = torch.from_numpy(np.power(np.float32(theta), exponent).astype(np.float32))
    pos = torch.as_tensor(list(positions), dtype=torch.float32)[:, None]
    angle = pos * freq[None, :]
    return torch.cos(angle).to(dtype), torch.sin(angle).to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Half-split rotation of each head: `x'[j] = x[j] c - x[j+D/2] s`,
    `x'[j+D/2] = x[j] s + x[j+D/2] c` (src/minillm/runtime.cpp:258-265).
    x is [T, heads, D]; cos, sin are [T, D/2]."""
    half = x.shape[-1] // 2
    left, right = x[..., :half], x[..., half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([left * c - right * s, left * s + right * c], dim=-1)


def qk_norm_rope(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, cos, sin) -> torch.Tensor:
    """Per head RMS norm over the D elements (same eps, one weight for all heads),
    then the rotation (src/minillm/runtime.cpp:256-257, :267-272).  x is [T, heads, D]."""
    return apply_rope(rms_norm(x, norm_weight, eps), cos, sin)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                     window: Optional[int] = None, scale: Optional[float] = None) -> torch.Tensor:
    """Scores, softmax and weighted sum for every query row, one row at a time.

    For query position p and head h (kv head `h // (Hq/Hkv)`), keys t in [lo, p]:
    `score_t = (q . k_t) * (1/sqrt(D))`; `m = max score`; `e_t = exp(score_t - m)`;
    `Z = sum e_t` in float64; `P_t = float(e_t / Z)`; `o = sum P_t v_t` in position
    order (src/minillm/runtime.cpp:283-310).  `lo` is 0 in the reference; with a
    window it is `max(0, p - window + 1)`.
    q is [T, Hq, D]; k, v are [T, Hkv, D]; returns [T, Hq, D]."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    out = torch.zeros_like(q)
    for p in range(T):
        lo = 0 if window is None else max(0, p - window + 1)
        for h in range(Hq):
            kv = h // group
            scores = (k[lo:p + 1, kv, :] @ q[p, h, :]) * scale
            e = torch.exp(scores - scores.max())
            z = e.to(torch.float64).sum()
            prob = (e.to(torch.float64) / z).to(q.dtype)
            out[p, h, :] = prob @ v[lo:p + 1, kv, :]
    return out


def attention_projections(n: torch.Tensor, w: dict, prefix: str, cfg: dict, cos, sin):
    """q, k, v of a layer: three products without bias (src/minillm/runtime.cpp:250-252),
    q and k normed per head and rotated, v untouched."""
    H = cfg["hidden_size"]
    Hq, Hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    D = cfg.get("head_dim") or H // Hq
    eps = cfg["rms_norm_eps"]
    dt = n.dtype
    T = n.shape[0]
    q = (n @ w[prefix + "self_attn.q_proj.weight"].to(dt).T).view(T, Hq, D)
    k = (n @ w[prefix + "self_attn.k_proj.weight"].to(dt).T).view(T, Hkv, D)
    v = (n @ w[prefix + "self_attn.v_proj.weight"].to(dt).T).view(T, Hkv, D)
    q = qk_norm_rope(q, w[prefix + "self_attn.q_norm.weight"], eps, cos, sin)
    k = qk_norm_rope(k, w[prefix + "self_attn.k_norm.weight"], eps, cos, sin)
    return q, k, v


def swiglu_mlp(n: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """`g = n Wg^T`, `u = n Wu^T`, `a = (g / (1 + exp(-g))) * u`, `d = a Wd^T`
    (src/minillm/runtime.cpp:323-335)."""
    dt = n.dtype
    g = n @ w[prefix + "mlp.gate_proj.weight"].to(dt).T
    u = n @ w[prefix + "mlp.up_proj.weight"].to(dt).T
    a = (g / (1.0 + torch.exp(-g))) * u
    return a @ w[prefix + "mlp.down_proj.weight"].to(dt).T


def decoder_layer(h: torch.Tensor, w: dict, layer: int, cfg: dict, cos, sin,
                  window: Optional[int], shared_kv=None):
    """One pre-norm block: `h += Wo attention(norm(h))`, `h += mlp(norm(h))`
    (src/minillm/runtime.cpp:245-337).  Returns the new h and this run's (k, v).
    With `shared_kv` the run attends with its own queries to another run's keys
    and values and writes none (not in the reference)."""
    prefix = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    dt = h.dtype
    n = rms_norm(h, w[prefix + "input_layernorm.weight"], eps)
    q, k, v = attention_projections(n, w, prefix, cfg, cos, sin)
    if shared_kv is not None:
        k, v = shared_kv
    o = causal_attention(q, k, v, window)
    h = h + o.reshape(h.shape[0], -1) @ w[prefix + "self_attn.o_proj.weight"].to(dt).T
    n2 = rms_norm(h, w[prefix + "post_attention_layernorm.weight"], eps)
    h = h + swiglu_mlp(n2, w, prefix)
    return h, (k, v)


def final_logits(h: torch.Tensor, w: dict, cfg: dict) -> torch.Tensor:
    """`logits = rms_norm(h, w_out_norm) @ W_out^T`; W_out is the embedding table
    when the checkpoint has no lm_head (src/minillm/runtime.cpp:338-351,
    src/minillm/qwen3_model.cpp:60-61)."""
    f = rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"])
    out = w["lm_head.weight"] if "lm_head.weight" in w else w["model.embed_tokens.weight"]
    return f @ out.to(h.dtype).T


# --------------------------------------------------------------------------- model
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], dtype=torch.float32,
            schedule: Optional[List[tuple]] = None, return_hidden: bool = False) -> torch.Tensor:
    """Logits [T, V] at every position of one whole sequence starting at position 0.

    `schedule` is a list of `(layer, kv_from)` runs; `kv_from` is None or the index
    of an earlier run whose keys and values this run reads.  Default: every layer
    once, in order (src/minillm/runtime.cpp:245)."""
    H = cfg["hidden_size"]
    D = cfg.get("head_dim") or H // cfg["num_attention_heads"]
    T = len(tokens)
    windows = layer_windows(cfg)
    if schedule is None:
        schedule = [(i, None) for i in range(cfg["num_hidden_layers"])]
    h = embedding(w["model.embed_tokens.weight"], tokens, dtype)
    cos, sin = rope_table(range(T), D, cfg.get("rope_theta", 10000.0), dtype)
    kept = []
    for layer, kv_from in schedule:
        shared = kept[kv_from] if kv_from is not None else None
        h, kv = decoder_layer(h, w, layer, cfg, cos, sin, windows[layer], shared)
        kept.append(kv)
    if return_hidden:
        return h
    return final_logits(h, w, cfg)


# --------------------------------------------------------------------------- sampling
def greedy(logits_row: torch.Tensor) -> int:
    """Largest logit, ties to the lowest id (src/minillm/cuda/ops.cu:166-201;
    CPU twin `std::max_element`, apps/mini_main.cpp:105)."""
    m = logits_row.max()
    return int(torch.nonzero(logits_row == m)[0, 0])


def uniform_for(seed: int, request: int, step: int) -> float:
    """The uniform number in [0, 1) that temperature sampling draws for
    (seed, request, step): a SplitMix64 finaliser over the three integers, top 53
    bits.  The reference samples greedily only (src/http_server.cpp:140-142); the
    draw is defined here and restated independently in the engine."""
    mask = (1 << 64) - 1
    x = (seed * 0x9E3779B97F4A7C15 + request * 0xBF58476D1CE4E5B9 + step * 0x94D049BB133111EB + 0x2545F4914F6CDD1D) & mask
    for _ in range(2):
        x ^= x >> 30
        x = (x * 0xBF58476D1CE4E5B9) & mask
        x ^= x >> 27
        x = (x * 0x94D049BB133111EB) & mask
        x ^= x >> 31
    return (x >> 11) / float(1 << 53)


def temperature_cdf(logits_row: torch.Tensor, temperature: float) -> torch.Tensor:
    """Cumulative distribution of `softmax(logits / T)`, exponentials in float32
    and sums in float64."""
    z = logits_row.to(torch.float32) / temperature
    e = torch.exp(z - z.max()).to(torch.float64)
    return torch.cumsum(e, 0) / e.sum()


def sample_temperature(logits_row: torch.Tensor, temperature: float, u: float) -> int:
    """Inverse-CDF draw: the first id whose cumulative probability exceeds u."""
    if temperature <= 0:
        return greedy(logits_row)
    cdf = temperature_cdf(logits_row, temperature)
    idx = int(torch.searchsorted(cdf, torch.tensor(u, dtype=torch.float64), right=True))
    return min(idx, logits_row.numel() - 1)
