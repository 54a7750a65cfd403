"""Builders of replay traces and the comparison of their logits with the plain implementation."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# a trace step also records, for the checker, which (request, position) each wanted row is
Step = dict


def whole(requests: Dict[str, List[int]]) -> List[Step]:
    """Each request alone and whole: one step with all its tokens, logits wanted everywhere."""
    steps = []
    for i, (rid, toks) in enumerate(requests.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def tail_one_by_one(requests: Dict[str, List[int]], tail: int = 32) -> List[Step]:
    """Each request alone: all but the last `tail` tokens in one step, then one token per step."""
    steps = []
    n = 0
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": n, "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        n += 1
        for j in range(head, len(toks)):
            steps.append({"step": n, "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
            n += 1
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def batched(requests: Dict[str, List[int]], batch: int, decode: Sequence[int]) -> List[Step]:
    """Batches of `batch` requests, one batch after another.  A batch's prompts (each request's tokens
    but its last `decode[i]`) go in one step; then every request that has tokens left brings one per
    step, so shorter requests end earlier."""
    ids = list(requests)
    steps = []
    n = 0
    for b0 in range(0, len(ids), batch):
        group = ids[b0:b0 + batch]
        heads = {}
        for k, rid in enumerate(group):
            d = decode[(b0 + k) % len(decode)]
            heads[rid] = max(1, len(requests[rid]) - d)
        entries = [{"id": r, "tokens": requests[r][:heads[r]], "want": list(range(heads[r]))} for r in group]
        done = [r for r in group if heads[r] == len(requests[r])]
        steps.append({"step": n, "entries": entries, "end": done})
        n += 1
        pos = dict(heads)
        live = [r for r in group if r not in done]
        while live:
            entries = [{"id": r, "tokens": [requests[r][pos[r]]], "want": [0]} for r in live]
            for r in live:
                pos[r] += 1
            done = [r for r in live if pos[r] == len(requests[r])]
            steps.append({"step": n, "entries": entries, "end": done})
            n += 1
            live = [r for r in live if r not in done]
    return steps


def chunked(requests: Dict[str, List[int]], cuts: Sequence[int]) -> List[Step]:
    """All requests together, each fed in pieces of `cuts` tokens (cycled) however long it is; requests
    that run out end earlier.  Not a pattern the replay program must take (its steps bring prompts or
    single tokens), but one the step function does: several tokens on top of a cache that is not empty."""
    pos = {r: 0 for r in requests}
    live = list(requests)
    steps = []
    k = 0
    while live:
        entries = []
        for r in live:
            n = min(cuts[k % len(cuts)], len(requests[r]) - pos[r])
            entries.append({"id": r, "tokens": requests[r][pos[r]:pos[r] + n], "want": list(range(n))})
            pos[r] += n
            k += 1
        done = [r for r in live if pos[r] == len(requests[r])]
        steps.append({"step": len(steps), "entries": entries, "end": done})
        live = [r for r in live if r not in done]
    return steps


def collect(steps: List[Step], outputs: Dict[int, torch.Tensor], requests: Dict[str, List[int]]) -> Dict[str, torch.Tensor]:
    """Put the wanted rows of every step back in place: request -> logits [len, vocab] (NaN where never wanted)."""
    vocab = next(iter(outputs.values())).shape[-1]
    got = {r: torch.full((len(t), vocab), float("nan")) for r, t in requests.items()}
    at = {r: 0 for r in requests}
    for st in steps:
        row = 0
        out = outputs.get(st["step"])
        for e in st["entries"]:
            for w in e["want"]:
                got[e["id"]][at[e["id"]] + w] = out[row]
                row += 1
            at[e["id"]] += len(e["tokens"])
        assert out is None or row == out.shape[0], f"step {st['step']}: {out.shape[0]} rows for {row} wanted"
    return got


def run_in_process(engine, steps: List[Step]) -> Dict[int, torch.Tensor]:
    from dlgo_b200.engine.replay import Replayer
    rp = Replayer(engine)
    outs = {}
    for st in steps:
        lg = rp.run_step(st)
        if lg is not None:
            outs[st["step"]] = lg.float().cpu().clone()
    assert rp.slots == {}, "the trace left requests open"
    return outs


def run_program(model_dir: str, dtype: str, steps: List[Step], out_dir: str, max_tokens: int, vocab: int,
                env: dict | None = None) -> Dict[int, torch.Tensor]:
    """Drive bin/trace_run as a user would: one line in, wait for `done <step>`, next line."""
    cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_dir, "--dtype", dtype,
           "--out", out_dir, "--max-tokens", str(max_tokens)]
    p = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True,
                         env={**os.environ, **(env or {})})
    try:
        for st in steps:
            p.stdin.write(json.dumps({k: st[k] for k in ("step", "entries", "end")}) + "\n")
            p.stdin.flush()
            line = p.stdout.readline().strip()
            assert line == f"done {st['step']}", f"expected 'done {st['step']}', got {line!r}"
        p.stdin.close()
        assert p.wait(timeout=120) == 0
    finally:
        if p.poll() is None:
            p.kill()
    outs = {}
    for st in steps:
        path = os.path.join(out_dir, f"{st['step']}.f32")
        wanted = sum(len(e["want"]) for e in st["entries"])
        if wanted:
            a = np.fromfile(path, dtype="<f4")
            assert a.size == wanted * vocab, f"{path}: {a.size} floats for {wanted} x {vocab}"
            outs[st["step"]] = torch.from_numpy(a.reshape(wanted, vocab).copy())
        else:
            assert not os.path.exists(path)
    return outs
