"""The plain implementation at sizes where its per-row attention loop would take hours.

Every part is `plain_qwen3`'s own function (embedding, norms, projections, rotation, gated
feed-forward, head); only the attention loop is replaced by a dense restatement of the same
definition (`plain_qwen3.causal_attention`: scores of keys `lo..p`, softmax, weighted sum),
computed for blocks of query rows at once, and tensors may live on a GPU.  It is still whole
sequences, no cache, no batching, and shares no code with the package under test.
`test_plain.py` checks it against the loop on a tiny model.

Run it in float64: it is then the truth that both precisions of the engine are measured
against.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch

import plain_qwen3 as P


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None,
                    scale: Optional[float] = None, block: int = 512) -> torch.Tensor:
    """q [T, Hq, D]; k, v [T, Hkv, D]; query row p reads keys max(0, p - window + 1) .. p
    (src/minillm/runtime.cpp:283-310)."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    out = torch.empty_like(q)
    for lo in range(0, T, block):
        hi = min(T, lo + block)
        first = 0 if window is None else max(0, lo - window + 1)
        qb = q[lo:hi].view(hi - lo, Hkv, group, D)
        s = torch.einsum("qkgd,tkd->kgqt", qb, k[first:hi]) * scale
        pos = torch.arange(lo, hi, device=q.device)[:, None]
        t = torch.arange(first, hi, device=q.device)[None, :]
        mask = t > pos
        if window is not None:
            mask = mask | (t < pos - window + 1)
        s = s.masked_fill(mask[None, None], float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[lo:hi] = torch.einsum("kgqt,tkd->qkgd", p, v[first:hi]).reshape(hi - lo, Hq, D)
    return out


def forward_rows(cfg: dict, w: Dict[str, torch.Tensor], tokens: Sequence[int], rows: Optional[Sequence[int]] = None,
                 dtype=torch.float64, device="cpu") -> torch.Tensor:
    """Logits at `rows` (default: all) of one whole sequence from position 0: the layers of
    `plain_qwen3.decoder_layer` in order, with the dense attention."""
    H = cfg["hidden_size"]
    D = cfg.get("head_dim") or H // cfg["num_attention_heads"]
    eps = cfg["rms_norm_eps"]
    windows = P.layer_windows(cfg)
    h = P.embedding(w["model.embed_tokens.weight"], tokens, dtype).to(device)
    cos, sin = (t.to(device) for t in P.rope_table(range(len(tokens)), D, cfg.get("rope_theta", 10000.0), dtype))
    for layer in range(cfg["num_hidden_layers"]):
        prefix = f"model.layers.{layer}."
        n = P.rms_norm(h, w[prefix + "input_layernorm.weight"], eps)
        q, k, v = P.attention_projections(n, w, prefix, cfg, cos, sin)
        o = dense_attention(q, k, v, windows[layer])
        h = h + o.reshape(h.shape[0], -1) @ w[prefix + "self_attn.o_proj.weight"].to(dtype).T
        h = h + P.swiglu_mlp(P.rms_norm(h, w[prefix + "post_attention_layernorm.weight"], eps), w, prefix)
    if rows is not None:
        h = h[torch.as_tensor(list(rows), dtype=torch.long, device=h.device)]
    return P.final_logits(h, w, cfg)
