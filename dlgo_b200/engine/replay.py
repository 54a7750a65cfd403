"""Trace replay: feed given token ids through the engine step by step and keep the logits.

The nearest things in the reference are its hand-driven ``Forward`` loops
(gpu_verify_main.go:68-76, models/llm/e2e_test.go:67-89).  A trace is a list of
steps; each step brings, per request, its next tokens and the places among them
whose logits are wanted, and names the requests that are finished after it.
Replay samples nothing and owns no model code: it calls :meth:`Engine.step`.
"""
from __future__ import annotations

import json
import os
from typing import Any, Callable, Dict, Iterable, Optional

import torch


class Replayer:
    def __init__(self, engine: Any):
        self.engine = engine
        self.slots: Dict[str, int] = {}

    def run_step(self, rec: dict) -> Optional[torch.Tensor]:
        """One step of a trace; returns the wanted logits ``[wanted, vocab]`` (device, fp32) or None."""
        entries = rec.get("entries", [])
        logits = None
        if entries:
            ids = [str(e["id"]) for e in entries]
            if len(set(ids)) != len(ids):
                raise ValueError(f"step {rec.get('step')}: a request appears twice")
            for rid in ids:
                if rid not in self.slots:
                    self.slots[rid] = self.engine.take_slot()
            tokens = [e["tokens"] for e in entries]
            want = [e.get("want", []) for e in entries]
            logits = self.engine.step([self.slots[r] for r in ids], tokens, want)
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in self.slots:
                self.engine.free_slot(self.slots.pop(rid))
        return logits


def replay_lines(engine: Any, lines: Iterable[str], out_dir: str, done: Callable[[Any], None]) -> None:
    """Run a trace given as JSON lines; write ``<out_dir>/<step>.f32`` for steps that want logits."""
    os.makedirs(out_dir, exist_ok=True)
    rp = Replayer(engine)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        logits = rp.run_step(rec)
        if logits is not None:
            arr = logits.float().cpu().contiguous().numpy().astype("<f4", copy=False)
            with open(os.path.join(out_dir, f"{rec['step']}.f32"), "wb") as f:
                f.write(arr.tobytes())
        done(rec["step"])
