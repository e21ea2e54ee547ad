#!/usr/bin/env python3
"""Benchmark of kvad_b200: GPT-2 small shapes, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

A "step" is one decode step of a batch of 8 sequences (512-token prompts, context 1024).
The one JSON line carries: `value` - decoded tokens a second, timed on the device over exactly K
steps with the chosen tokens fed back on the device; `e2e` - the same through `Engine.generate`,
host token ids in and out every step; `prefill` - one step of 2 x 1024 prompt tokens; `roofline` -
the decode step's bytes (every weight once + the live cache) over its time, against the measured
copy bandwidth; `points` - decoding at batch 1 and 64.  Weights are random (seeded), token ids
uniform-random (seeded): there is no dataset and no checkpoint here.

bisand/kvad is a Rust workspace without a Python package, so `--impl reference` reports itself
unavailable.  This library runs on one GPU: `--gpus N` with N > 1 says so and exits with 2.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GPT2_SMALL = dict(model_type="gpt2", n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                  n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new",
                  scale_attn_by_inverse_layer_idx=False, tie_word_embeddings=True)
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
SMI_QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            out = dict(FALLBACK_PEAKS)
            out.update({k: float(v) for k, v in p.items() if k in FALLBACK_PEAKS and v})
            return out, "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while a timed region runs."""

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", "0"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            self.thread.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (IndexError, ValueError):
                continue
            for name, cell in zip(names, r[5:9]):
                if cell.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def random_prompts(n, length, vocab, seed):
    import numpy as np
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, length).tolist() for _ in range(n)]


def decode_point(engine, batch, prompt_len, steps, warmup, seed, clock=False, sampled=False):
    """Device-timed decoding: prompts in one step, `warmup` untimed steps, then exactly `steps` steps.
    `sampled`: every request draws with temperature 0.7, top-k 40, top-p 0.95 instead of taking the best token."""
    import torch
    from kvad_b200 import StepEntry
    from kvad_b200.sampling import RequestSampler, SamplingParams

    prompts = random_prompts(batch, prompt_len, engine.vocab_size, seed)
    slots = [engine.open() for _ in prompts]
    samplers = [RequestSampler(SamplingParams(0.7, 40, 0.95, seed + i)) for i in range(batch)] if sampled else None
    try:
        logits = engine.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)])
        first = logits.argmax(dim=-1).tolist()
        hist = engine.decode_run(slots, first, warmup, samplers)
        nxt = hist[-1].tolist()
        torch.cuda.synchronize()
        k0, start, end = engine.graph_kernels, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler() if clock else None
        if sampler:
            sampler.__enter__()
        torch.cuda.synchronize()
        start.record()
        engine.decode_run(slots, nxt, steps, samplers)
        end.record()
        torch.cuda.synchronize()
        if sampler:
            sampler.__exit__()
        ms = start.elapsed_time(end)
        launches = engine.graph_kernels - k0
        mean_ctx = prompt_len + 1 + warmup + (steps - 1) / 2.0
    finally:
        for s in slots:
            engine.close(s)
    return {"tok_s": batch * steps / (ms * 1e-3), "ms_per_step": ms / steps, "launches": launches,
            "mean_ctx": mean_ctx, "clocks": sampler.summary() if sampler else None}


def prefill_point(engine, n_seqs, length, iters, warmup, seed):
    import torch
    from kvad_b200 import StepEntry

    prompts = random_prompts(n_seqs, length, engine.vocab_size, seed)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=engine.device)
    times = []
    for i in range(warmup + iters):
        slots = [engine.open() for _ in prompts]
        flush.zero_()                                   # L2 flushed between iterations
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)])
        end.record()
        torch.cuda.synchronize()
        for s in slots:
            engine.close(s)
        if i >= warmup:
            times.append(start.elapsed_time(end))
    return statistics.median(times)


def prefill_flops(cfg, n_layers, n_seqs, length, wanted_rows):
    e, i, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    t = n_seqs * length
    per_layer = 2 * t * (3 * e * e + e * e + 2 * e * i) + n_seqs * 2 * e * length * (length + 1)
    return n_layers * per_layer + 2 * wanted_rows * e * v


def decode_bytes(engine, batch, mean_ctx):
    """What one decode step has to read: every weight it uses once, and the cache of the live requests."""
    import torch
    elem = torch.empty((), dtype=engine.dtype).element_size()
    weights = engine.model.weight_bytes()
    pos = engine.model.embedding.position
    if pos is not None and pos.table() is not None:     # of the position table only one row per sequence is read
        weights -= pos.table().numel() * elem
        weights += batch * pos.table().shape[1] * elem
    cache = batch * mean_ctx * engine.cache.layout.bytes_per_token(elem)
    return weights + cache


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--layers", type=int, default=GPT2_SMALL["n_layer"], help="fewer layers than GPT-2 small has (named in config)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profiling)")
    ap.add_argument("--phase", default="all", choices=["all", "prefill"], help="`prefill`: only the 2 x 1024-token prefill (profiling)")
    ap.add_argument("--skip-points", action="store_true", help="leave out batch 1 / 64, prefill and e2e (quick runs)")
    ap.add_argument("--sampling", default="greedy", choices=["greedy", "sampled"],
                    help="`sampled`: the timed decode steps draw with temperature 0.7, top-k 40, top-p 0.95")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "bisand/kvad is a Rust workspace (no setup.py/pyproject; needs cargo, which this image lacks): "
                          "pip cannot install it offline"}))
        return 0
    if args.gpus != 1:
        print(f"kvad_b200 runs on one GPU; --gpus {args.gpus} is not built (multi-GPU work is out of this library's scope)")
        return 2
    warmup = max(3, args.warmup)
    cfg = dict(GPT2_SMALL)
    n_layers_full = cfg["n_layer"]
    cfg["n_layer"] = args.layers
    if args.prompt_len + 1 + warmup + args.steps > cfg["n_positions"]:
        print(f"prompt {args.prompt_len} + warm-up {warmup} + steps {args.steps} exceed the context of {cfg['n_positions']}", file=sys.stderr)
        return 1

    import torch
    from kvad_b200 import Engine, write_random_model
    from kvad_b200.ops import launch_count

    pk, pk_src = peaks()
    with tempfile.TemporaryDirectory(prefix="kvad_b200-bench-") as d:
        write_random_model(d, cfg, seed=0)
        engine = Engine.from_pretrained(d, args.dtype, max_tokens=max(64, args.batch) * cfg["n_positions"])
    engine.use_graphs = not args.no_graphs
    print(f"[bench] {engine.describe()}", file=sys.stderr)

    if args.phase == "prefill":
        t_ms = prefill_point(engine, 2, 1024, iters=3, warmup=3, seed=3)
        fl = prefill_flops(cfg, args.layers, 2, 1024, 2)
        print(json.dumps({"phase": "prefill", "tokens": 2048, "ms": round(t_ms, 4), "tokens_per_s": round(2048 / (t_ms * 1e-3), 1),
                          "tflops": round(fl / (t_ms * 1e-3) / 1e12, 2), "frac": round(fl / (t_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                          "of": pk_src}))
        return 0
    main_pt = decode_point(engine, args.batch, args.prompt_len, args.steps, warmup, seed=1, clock=True, sampled=args.sampling == "sampled")
    bytes_step = decode_bytes(engine, args.batch, main_pt["mean_ctx"])
    achieved = bytes_step / (main_pt["ms_per_step"] * 1e-3) / 1e9
    out = {
        "metric": "decode tok/s at batch 8, GPT-2 small (124M), 512-token prompts",
        "value": round(main_pt["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_pt["ms_per_step"], 5), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: seeded uniform-random token ids, seeded random weights",
        "config": {"model": "gpt2-small-124M", "global_batch": args.batch, "seq_len": cfg["n_positions"],
                   "parallelism": "single-gpu", "prompt_len": args.prompt_len, "decode_steps": args.steps,
                   "n_layer": n_layers_full, "n_layer_run": args.layers, "n_embd": cfg["n_embd"], "n_head": cfg["n_head"],
                   "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"],
                   "sampling": "greedy" if args.sampling == "greedy" else "temperature 0.7, top-k 40, top-p 0.95", "weights": "random seed 0", "cache_page_tokens": 64,
                   "l2": "inputs larger than L2: a step streams %.0f MB" % (bytes_step / 1e6),
                   "peaks": pk_src},
        "gpu_launches": int(main_pt["launches"]),
        "clocks": main_pt["clocks"],
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_src, "bytes_per_step": int(bytes_step)},
    }

    if not args.skip_points:
        # end to end through the public entry point: host token ids in, host token ids out, every step
        prompts = random_prompts(args.batch, args.prompt_len, engine.vocab_size, seed=2)
        engine.generate(prompts, max_tokens=4, temperature=0.0, stop_token_ids=[])        # warm
        h0, d0 = engine.h2d_bytes, engine.d2h_bytes
        e2e_steps = min(args.steps, 128)
        _, stats = engine.generate(prompts, max_tokens=e2e_steps + 1, temperature=0.0, stop_token_ids=[], return_stats=True)
        n_dec = stats.steps - 1
        out["e2e"] = {"value": round(args.batch * n_dec / stats.decode_secs, 1), "unit": "tokens/s",
                      "h2d_bytes_per_step": int((engine.h2d_bytes - h0) / stats.steps),
                      "d2h_bytes_per_step": int((engine.d2h_bytes - d0) / stats.steps),
                      "steps": n_dec, "api": "Engine.generate"}

        t_ms = prefill_point(engine, 2, 1024, iters=5, warmup=3, seed=3)
        fl = prefill_flops(cfg, args.layers, 2, 1024, 2)
        peak_fl = pk["bf16_tflops"] * 1e12
        out["prefill"] = {"value": round(2048 / (t_ms * 1e-3), 1), "tokens": 2048, "ms": round(t_ms, 4),
                          "frac": round(fl / (t_ms * 1e-3) / peak_fl, 4), "tflops": round(fl / (t_ms * 1e-3) / 1e12, 2),
                          "of": pk_src}
        points = {}
        for b in (1, 64):
            pt = decode_point(engine, b, args.prompt_len, min(args.steps, 128), warmup, seed=10 + b)
            points[f"decode_b{b}"] = round(pt["tok_s"], 1)
            by = decode_bytes(engine, b, pt["mean_ctx"])
            points[f"decode_b{b}_hbm_frac"] = round(by / (pt["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        pt = decode_point(engine, args.batch, args.prompt_len, min(args.steps, 128), warmup, seed=30, sampled=True)
        points[f"decode_b{args.batch}_sampled"] = round(pt["tok_s"], 1)      # temperature 0.7, top-k 40, top-p 0.95
        out["points"] = points

    from kvad_b200.csrc import build
    out["loaded_libraries"] = [os.path.basename(p) for p in build.loaded_paths()]
    engine.cache.book.check_all_free()
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
