"""Builds replay traces, runs `bin/trace_run` on them as a user would (a child
process fed over a pipe, one step at a time), and gathers logits by (request,
position)."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def round64(n: int) -> int:
    return (n + 63) // 64 * 64


def whole(requests: Dict[str, List[int]]) -> List[dict]:
    """Each request alone, all tokens in one step."""
    return [{"step": i, "entries": [{"id": k, "tokens": t, "want": list(range(len(t)))}], "end": [k]}
            for i, (k, t) in enumerate(requests.items())]


def last_32_one_by_one(requests: Dict[str, List[int]]) -> List[dict]:
    steps = []
    for k, t in requests.items():
        cut = max(1, len(t) - 32)
        steps.append({"entries": [{"id": k, "tokens": t[:cut], "want": list(range(cut))}], "end": []})
        for p in range(cut, len(t)):
            steps.append({"entries": [{"id": k, "tokens": [t[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [k]
    return [dict(s, step=i) for i, s in enumerate(steps)]


def portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (16, 7, 2, 5, 2, 33, 1, 3, 2, 64)) -> List[dict]:
    """One request at a time, cut into portions of changing size, down to two tokens."""
    steps = []
    for k, t in requests.items():
        pos, i = 0, 0
        while pos < len(t):
            n = min(sizes[i % len(sizes)], len(t) - pos)
            steps.append({"entries": [{"id": k, "tokens": t[pos:pos + n], "want": list(range(n))}], "end": []})
            pos += n
            i += 1
        steps[-1]["end"] = [k]
    return [dict(s, step=i) for i, s in enumerate(steps)]


def mixed(requests: Dict[str, List[int]], seed: int, live_limit: int = 4) -> List[dict]:
    """Up to `live_limit` live requests; each step takes some of them, gives prompt
    portions of changing size to those still in their prompt (the first two thirds of
    a request) and single tokens to the others; a request may sit a step out; a
    finished request ends and the next one starts, so its pages are used again."""
    rng = random.Random(seed)
    waiting = list(requests)
    live: Dict[str, int] = {}
    steps = []
    while waiting or live:
        while waiting and len(live) < live_limit and (not live or rng.random() < 0.6):
            live[waiting.pop(0)] = 0
        chosen = [k for k in live if rng.random() < 0.8] or [rng.choice(list(live))]
        entries, end = [], []
        for k in chosen:
            t, pos = requests[k], live[k]
            prompt = len(t) * 2 // 3
            n = min(rng.choice([2, 3, 5, 8, 16, 29, 70, 130]), prompt - pos) if pos < prompt else 1
            entries.append({"id": k, "tokens": t[pos:pos + n], "want": list(range(n))})
            live[k] = pos + n
            if live[k] == len(t):
                end.append(k)
        for k in end:
            del live[k]
        steps.append({"entries": entries, "end": end})
    return [dict(s, step=i) for i, s in enumerate(steps)]


def max_live_tokens(trace: List[dict]) -> int:
    held: Dict[str, int] = {}
    peak = 0
    for step in trace:
        for e in step["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(round64(n) for n in held.values()))
        for k in step["end"]:
            held.pop(k, None)
    return peak


def run_trace(model_dir: str, dtype: str, trace: List[dict], out_dir: str, vocab: int,
              max_tokens: int = 0, env: dict = None, timeout: float = 600.0,
              page_size: int = 0) -> Dict[Tuple[str, int], torch.Tensor]:
    """Feeds the trace to bin/trace_run, waiting for `done <step>` after each line."""
    max_tokens = max_tokens or max_live_tokens(trace)
    proc = subprocess.Popen([sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
                             "--max-tokens", str(max_tokens)] + (["--page-size", str(page_size)] if page_size else []),
                            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
    try:
        for step in trace:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            answer = proc.stdout.readline().strip()
            assert answer == f"done {step['step']}", f"expected 'done {step['step']}', got {answer!r}"
        proc.stdin.close()
        assert proc.wait(timeout=timeout) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    logits: Dict[Tuple[str, int], torch.Tensor] = {}
    position: Dict[str, int] = {}
    for step in trace:
        wanted = [(e["id"], position.get(e["id"], 0) + w) for e in step["entries"] for w in e.get("want", [])]
        for e in step["entries"]:
            position[e["id"]] = position.get(e["id"], 0) + len(e["tokens"])
        path = os.path.join(out_dir, f"{step['step']}.f32")
        if not wanted:
            assert not os.path.exists(path)
            continue
        data = np.fromfile(path, dtype="<f4")
        assert data.size == len(wanted) * vocab, f"step {step['step']}: {data.size} floats for {len(wanted)} rows"
        rows = torch.from_numpy(data.reshape(len(wanted), vocab).copy())
        for key, row in zip(wanted, rows):
            logits[key] = row
        for k in step["end"]:
            position.pop(k, None)
    return logits


def stack(logits: Dict[Tuple[str, int], torch.Tensor], name: str, length: int) -> torch.Tensor:
    return torch.stack([logits[(name, p)] for p in range(length)])
