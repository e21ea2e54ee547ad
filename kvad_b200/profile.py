"""An opt-in table of where a run's device time goes, kernel call by kernel call.

With `KVAD_PROFILE=1` every call of an `Ops` method that launches kernels is
bracketed by two CUDA events on the launching stream; steps are then launched
kernel by kernel (no CUDA graphs, or the events would not be reached), and at
exit one table goes to standard error: per operation and shape class the
number of calls, the total, mean and share of the device time.  Times taken
this way include the gaps that programmatic dependent launch would close, so
they say where the time goes, not how long a captured step takes.

bisand/kvad keeps the same kind of table behind `KVAD_PROFILE`
(crates/gpu/src/prof.rs:54-87: a label and an elapsed time per scope, summed
and printed at the end).
"""
from __future__ import annotations

import atexit
import functools
import os
import sys

import torch

#: methods of `Ops` that launch kernels, and the argument whose leading size names the shape class
_TIMED = {"embed": 4, "layernorm": 4, "linear": 3, "kv_store": 0, "attention": 0, "attention_prefill": 0, "attention_prompt": 0, "attention_decode_sums": 0,
          "attention_decode": 0, "argmax": 0, "sample": 0}

_records: list = []       # (label, start event, end event)
_registered = False


def enabled() -> bool:
    return os.environ.get("KVAD_PROFILE", "0") == "1"


def _label(name: str, args, kwargs) -> str:
    t = args[_TIMED[name]] if len(args) > _TIMED[name] else None
    rows = int(t.shape[0]) if isinstance(t, torch.Tensor) and t.dim() >= 1 else 0
    if name == "linear":
        weight = args[1]
        epi = args[4] if len(args) > 4 else kwargs.get("epilogue", "store")
        return f"linear {rows}x{weight.shape[0]}x{weight.shape[1]} {epi}"
    return f"{name} rows={rows}"


def instrument(ops) -> None:
    """Wraps the kernel-launching methods of one `Ops` object (called by `Ops.__init__` when profiling is on)."""
    global _registered
    for name in _TIMED:
        fn = getattr(ops, name)

        def timed(*args, __fn=fn, __name=name, **kwargs):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = __fn(*args, **kwargs)
            end.record()
            _records.append((_label(__name, args, kwargs), start, end))
            return out

        setattr(ops, name, functools.wraps(fn)(timed))
    if not _registered:
        atexit.register(report)
        _registered = True


def table() -> list[tuple[str, int, float]]:
    """(label, calls, total microseconds), largest total first.  Waits for the device."""
    torch.cuda.synchronize()
    sums: dict[str, list] = {}
    for label, start, end in _records:
        row = sums.setdefault(label, [0, 0.0])
        row[0] += 1
        row[1] += start.elapsed_time(end) * 1e3
    return sorted(((k, n, us) for k, (n, us) in sums.items()), key=lambda r: -r[2])


def report(file=None) -> None:
    if not _records:
        return
    file = file or sys.stderr
    rows = table()
    total = sum(us for _, _, us in rows) or 1.0
    print(f"[kvad_b200] device time by operation (KVAD_PROFILE=1, kernel-by-kernel launches): {total / 1e3:.2f} ms", file=file)
    print(f"{'operation':48s} {'calls':>7s} {'total ms':>10s} {'mean us':>9s} {'share':>7s}", file=file)
    for label, n, us in rows:
        print(f"{label:48s} {n:7d} {us / 1e3:10.3f} {us / n:9.2f} {100 * us / total:6.1f}%", file=file)
    _records.clear()
