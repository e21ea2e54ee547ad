"""Trace replay: feeds given token ids through the engine step by step and
writes logits.  Nothing is sampled.

It drives the same `Engine.step` that generation uses - the same model,
cache and kernels - and owns nothing but the mapping from a trace's request
ids to cache slots.  bisand/kvad's nearest relatives are its hand-driven
session example (crates/gpu/examples/replay.rs:56-135) and the spy session
that records pass sizes and logits (crates/llm/tests/trained_models.rs:318-352).

Input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

`entries`: each request's next tokens and the places among them whose logits
are wanted; `end`: requests that are finished after this step.  For a step in
which something is wanted, `<out>/<step>.f32` holds the logits as
little-endian float32 `[wanted, vocab]`, in the order of the entries and of
their `want` lists.  After every step a line `done <step>` is printed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np

from .batch import StepEntry


class Replayer:
    def __init__(self, engine, out_dir: str):
        self.engine = engine
        self.out_dir = out_dir
        self.slots: dict[str, int] = {}
        os.makedirs(out_dir, exist_ok=True)

    def run_step(self, record: dict) -> Optional[str]:
        """Runs one step; returns the path written, if any."""
        step = record.get("step")
        entries = []
        for e in record.get("entries", []):
            rid = str(e["id"])
            if rid not in self.slots:
                self.slots[rid] = self.engine.open()
            entries.append(StepEntry(self.slots[rid], [int(t) for t in e["tokens"]],
                                     [int(w) for w in e.get("want", [])]))
        path = None
        if entries:
            logits = self.engine.step(entries)
            if logits.shape[0] > 0:
                path = os.path.join(self.out_dir, f"{step}.f32")
                logits.detach().cpu().numpy().astype("<f4", copy=False).tofile(path)
        for rid in record.get("end", []):
            slot = self.slots.pop(str(rid), None)
            if slot is not None:
                self.engine.close(slot)
        return path

    def run(self, lines: IO[str], out: IO[str] = sys.stdout) -> int:
        n = 0
        for line in lines:
            line = line.strip()
            if not line:
                continue
            record = json.loads(line)
            self.run_step(record)
            print(f"done {record.get('step')}", file=out, flush=True)
            n += 1
        self.close_all()
        return n

    def close_all(self) -> None:
        """Gives back what requests still hold that no step has ended."""
        for slot in self.slots.values():
            self.engine.close(slot)
        self.slots.clear()


def main(argv=None) -> int:
    import argparse

    p = argparse.ArgumentParser(prog="trace_run", description="Feed given tokens through a model step by step; write logits.")
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    args = p.parse_args(argv)

    from .engine import Engine

    engine = Engine.from_pretrained(args.model, args.dtype, max_tokens=args.max_tokens)
    print(f"[kvad_b200] {engine.describe()}", file=sys.stderr, flush=True)
    Replayer(engine, args.out).run(sys.stdin)
    return 0
