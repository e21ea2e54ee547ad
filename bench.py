#!/usr/bin/env python3
"""Benchmark of kvad_b200: GPT-2 shapes, random weights, one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W]

A "step" is one decode step of a batch of 8 sequences (512-token prompts, context 1024).
The one JSON line carries: `value` - decoded tokens a second, timed on the device over exactly K
steps with the chosen tokens fed back on the device (the median of `--rounds` such regions, each
after its own prefill and W warm-up steps; `rounds` holds min / median / max); `e2e` - the same
through `Engine.generate`, host token ids in and out every step; `prefill` - one step of 2 x 1024
prompt tokens; `roofline` - the decode step's bytes (every weight once + the live cache) over its
time, against the measured copy bandwidth; `points` - decoding at batch 1 and 64, sampled decoding,
the 32-bit engine, and GPT-2 medium's and XL's workloads (`--points small` leaves those two out); `checked` - the
bfloat16 engine's logits at the prompts' ends against the 32-bit engine's on the same weights.
Weights are random (seeded), token ids uniform-random (seeded): there is no dataset and no
checkpoint here.

Fractions: decode points divide bytes/s by the measured copy bandwidth; prefill divides FLOP/s by
the measured bf16 matrix peak taken as a burst (`frac`; a prefill step is a burst of a millisecond)
and also by the sustained one (`frac_sustained`).  The 32-bit engine's prefill has no tensor-core
peak to stand against and is reported as TFLOP/s only.

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

GPT2 = {
    "small": dict(model_type="gpt2", n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                  n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new",
                  scale_attn_by_inverse_layer_idx=False, tie_word_embeddings=True),
    "medium": dict(model_type="gpt2", n_layer=24, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257,
                   n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "xl": dict(model_type="gpt2", n_layer=48, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257,
               n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
}
GPT2_SMALL = GPT2["small"]
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
    """Samples nvidia-smi clocks and throttle reasons of THIS process's GPU while timed regions run (query only)."""

    def __init__(self):
        self.rows, self.proc = [], None

    def __enter__(self):
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
            which = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
        except Exception:  # noqa: BLE001
            which = "0"
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={SMI_QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", which], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
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
            time.sleep(0.1)
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
    lengths = length if isinstance(length, (list, tuple)) else [length] * n
    return [rng.integers(0, vocab, int(k)).tolist() for k in lengths]


def spread(values, digits=1):
    return {"n": len(values), "min": round(min(values), digits), "median": round(statistics.median(values), digits),
            "max": round(max(values), digits)}


def decode_round(engine, prompts, steps, warmup, sampled, seed):
    """One timed region: the prompts in one step, `warmup` untimed decode steps, then exactly `steps` steps on the device."""
    import torch
    from kvad_b200 import StepEntry
    from kvad_b200.sampling import RequestSampler, SamplingParams

    slots = [engine.open() for _ in prompts]
    samplers = [RequestSampler(SamplingParams(0.7, 40, 0.95, seed + i)) for i in range(len(prompts))] if sampled else None
    try:
        logits = engine.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)])
        first = logits.argmax(dim=-1).tolist()
        hist = engine.decode_run(slots, first, warmup, samplers)
        nxt = hist[-1].tolist()
        torch.cuda.synchronize()
        k0, start, end = engine.graph_kernels, torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.decode_run(slots, nxt, steps, samplers)
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end), engine.graph_kernels - k0
    finally:
        for s in slots:
            engine.close(s)


def decode_point(engine, batch, prompt_len, steps, warmup, seed, rounds=5, sampled=False):
    """Device-timed decoding over `rounds` regions; the first region (which also captures the step's graph) is discarded."""
    prompts = random_prompts(batch, prompt_len, engine.vocab_size, seed)
    decode_round(engine, prompts, min(steps, 4), warmup, sampled, seed)
    ms, launches = [], 0
    for _ in range(rounds):
        t, launches = decode_round(engine, prompts, steps, warmup, sampled, seed)
        ms.append(t)
    lens = [len(p) for p in prompts]
    mean_ctx = sum(lens) / len(lens) + 1 + warmup + (steps - 1) / 2.0
    med = statistics.median(ms)
    return {"tok_s": batch * steps / (med * 1e-3), "ms_per_step": med / steps, "launches": launches, "mean_ctx": mean_ctx,
            "tok_s_rounds": spread([batch * steps / (t * 1e-3) for t in ms])}


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
    return times


def prefill_flops(cfg, n_layers, lengths, wanted_rows):
    e, i, v = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    t = sum(lengths)
    per_layer = 2 * t * (3 * e * e + e * e + 2 * e * i) + sum(2 * e * n * (n + 1) for n in lengths)
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


def hbm_frac(engine, batch, pt, pk):
    return decode_bytes(engine, batch, pt["mean_ctx"]) / (pt["ms_per_step"] * 1e-3) / 1e9 / pk["hbm_gbs"]


def prefill_summary(times_ms, flops, tokens, pk, pk_src, tensor_cores=True):
    t = statistics.median(times_ms)
    out = {"value": round(tokens / (t * 1e-3), 1), "tokens": tokens, "ms": round(t, 4), "ms_rounds": spread(times_ms, 4),
           "tflops": round(flops / (t * 1e-3) / 1e12, 2)}
    if tensor_cores:
        out["frac"] = round(flops / (t * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        out["frac_sustained"] = round(flops / (t * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        out["of"] = pk_src + " bf16 peak: frac against the burst figure, frac_sustained against the sustained one"
    return out


def self_check(engine, ref, cfg, seed):
    """The bfloat16 engine's logits at the ends of two 512-token prompts against the 32-bit engine on the same weights."""
    from kvad_b200 import StepEntry

    prompts = random_prompts(2, 512, cfg["vocab_size"], seed)
    rows = []
    for e in (engine, ref):
        slots = [e.open() for _ in prompts]
        rows.append(e.step([StepEntry(s, p, (len(p) - 1,)) for s, p in zip(slots, prompts)]).float().clone())
        for s in slots:
            e.close(s)
    return float((rows[0] - rows[1]).abs().max() / rows[1].abs().max())


def build_engine(model_dir, cfg, dtype, max_tokens, no_graphs=False):
    from kvad_b200 import Engine
    engine = Engine.from_pretrained(model_dir, dtype, max_tokens=max_tokens)
    if no_graphs:
        engine.use_graphs = False
    return engine


def large_points(points, pk, pk_src, args):
    """BASELINE's workloads for GPT-2 medium (8 prompts of 64..896 tokens, 128 steps) and XL (prefill 2 x 1024,
    decode at batch 1 / 8 / 64 from 512-token prompts for 128 steps), random weights."""
    import numpy as np
    import torch
    from kvad_b200 import write_random_model

    for name in ("medium", "xl"):
        cfg = GPT2[name]
        with tempfile.TemporaryDirectory(prefix=f"kvad_b200-bench-{name}-") as d:
            t0 = time.time()
            write_random_model(d, cfg, seed=0)
            engine = build_engine(d, cfg, "bfloat16", 64 * cfg["n_positions"])
        print(f"[bench] {name}: {engine.describe().splitlines()[1]} (made in {time.time() - t0:.0f} s)", file=sys.stderr)
        if name == "medium":
            # 64..892 rather than ..896: the longest prompt, 3 warm-up steps and 128 timed ones must fit 1024 positions
            lens = [int(x) for x in np.random.default_rng(4).integers(64, 893, 8)]
            pt = decode_point(engine, 8, lens, 128, 3, seed=40, rounds=args.rounds)
            points["medium_decode_b8"] = round(pt["tok_s"], 1)
            points["medium_decode_b8_hbm_frac"] = round(hbm_frac(engine, 8, pt, pk), 4)
            points["medium_decode_b8_rounds"] = pt["tok_s_rounds"]
        else:
            times = prefill_point(engine, 2, 1024, iters=args.rounds, warmup=3, seed=3)
            points["xl_prefill"] = prefill_summary(times, prefill_flops(cfg, cfg["n_layer"], [1024, 1024], 2), 2048, pk, pk_src)
            for b in (1, 8, 64):
                pt = decode_point(engine, b, 512, 128, 3, seed=50 + b, rounds=args.rounds)
                points[f"xl_decode_b{b}"] = round(pt["tok_s"], 1)
                points[f"xl_decode_b{b}_hbm_frac"] = round(hbm_frac(engine, b, pt, pk), 4)
        engine.cache.book.check_all_free()
        del engine
        torch.cuda.empty_cache()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--rounds", type=int, default=5, help="timed regions per point (median, min and max are reported)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512)
    ap.add_argument("--model", default="small", choices=sorted(GPT2), help="layer sizes of the timed model; the headline is `small` (profiling runs name another)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config); 0: all of them")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel (for profiling)")
    ap.add_argument("--phase", default="all", choices=["all", "prefill"], help="`prefill`: only the 2 x 1024-token prefill (profiling)")
    ap.add_argument("--points", default="large", choices=["none", "small", "large"],
                    help="`none`: only the headline; `small`: GPT-2 small's other points; `large` (default): also GPT-2 medium's and "
                         "XL's workloads (0.7 and 3.1 GB of random weights: about half a minute more)")
    ap.add_argument("--skip-points", action="store_true", help="the same as --points none")
    ap.add_argument("--sampling", default="greedy", choices=["greedy", "sampled"],
                    help="`sampled`: the timed decode steps draw with temperature 0.7, top-k 40, top-p 0.95")
    args = ap.parse_args()
    if args.skip_points:
        args.points = "none"

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "bisand/kvad is a Rust workspace (no setup.py/pyproject; needs cargo, which this image lacks): "
                          "pip cannot install it offline"}))
        return 0
    if args.gpus != 1:
        print(f"kvad_b200 runs on one GPU; --gpus {args.gpus} is not built (multi-GPU work is out of this library's scope)")
        return 2
    warmup = max(3, args.warmup)
    cfg = dict(GPT2[args.model])
    n_layers_full = cfg["n_layer"]
    args.layers = args.layers or n_layers_full
    cfg["n_layer"] = args.layers
    if args.prompt_len + 1 + warmup + args.steps > cfg["n_positions"]:
        print(f"prompt {args.prompt_len} + warm-up {warmup} + steps {args.steps} exceed the context of {cfg['n_positions']}", file=sys.stderr)
        return 1

    import torch
    from kvad_b200 import write_random_model

    pk, pk_src = peaks()
    tmp = tempfile.TemporaryDirectory(prefix="kvad_b200-bench-")
    model_dir = tmp.name
    write_random_model(model_dir, cfg, seed=0)
    engine = build_engine(model_dir, cfg, args.dtype, max(64, args.batch) * cfg["n_positions"], args.no_graphs)
    print(f"[bench] {engine.describe()}", file=sys.stderr)
    flops_2x1024 = prefill_flops(cfg, args.layers, [1024, 1024], 2)

    if args.phase == "prefill":
        times = prefill_point(engine, 2, 1024, iters=3, warmup=3, seed=3)
        print(json.dumps({"phase": "prefill", **prefill_summary(times, flops_2x1024, 2048, pk, pk_src, args.dtype == "bfloat16")}))
        return 0

    with ClockSampler() as clock:
        main_pt = decode_point(engine, args.batch, args.prompt_len, args.steps, warmup, seed=1, rounds=args.rounds,
                               sampled=args.sampling == "sampled")
    bytes_step = decode_bytes(engine, args.batch, main_pt["mean_ctx"])
    achieved = bytes_step / (main_pt["ms_per_step"] * 1e-3) / 1e9
    clocks = clock.summary()
    if clocks["sm_mhz"]:
        clocks["ms_per_step_x_sm_mhz"] = round(main_pt["ms_per_step"] * clocks["sm_mhz"], 2)
    out = {
        "metric": "decode tok/s at batch %d, %s, %d-token prompts"
                  % (args.batch, {"small": "GPT-2 small (124M)", "medium": "GPT-2 medium (355M)", "xl": "GPT-2 XL (1.5B)"}[args.model], args.prompt_len),
        "value": round(main_pt["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(main_pt["ms_per_step"], 5), "rounds": main_pt["tok_s_rounds"], "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
        "data": "synthetic: seeded uniform-random token ids, seeded random weights",
        "config": {"model": {"small": "gpt2-small-124M", "medium": "gpt2-medium-355M", "xl": "gpt2-xl-1.5B"}[args.model], "global_batch": args.batch, "seq_len": cfg["n_positions"],
                   "parallelism": "single-gpu", "prompt_len": args.prompt_len, "decode_steps": args.steps,
                   "n_layer": n_layers_full, "n_layer_run": args.layers, "n_embd": cfg["n_embd"], "n_head": cfg["n_head"],
                   "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"],
                   "sampling": "greedy" if args.sampling == "greedy" else "temperature 0.7, top-k 40, top-p 0.95", "weights": "random seed 0", "cache_page_tokens": 64,
                   "l2": "inputs larger than L2: a step streams %.0f MB" % (bytes_step / 1e6),
                   "peaks": pk_src},
        "gpu_launches": int(main_pt["launches"]),
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_src + " copy bandwidth", "bytes_per_step": int(bytes_step)},
    }

    if args.points != "none":
        # end to end through the public entry point: host token ids in, host token ids out, every step
        prompts = random_prompts(args.batch, args.prompt_len, engine.vocab_size, seed=2)
        engine.generate(prompts, max_tokens=4, temperature=0.0, stop_token_ids=[])        # warm
        e2e_steps, e2e_vals = min(args.steps, 128), []
        for _ in range(args.rounds):
            h0, d0 = engine.h2d_bytes, engine.d2h_bytes
            _, stats = engine.generate(prompts, max_tokens=e2e_steps + 1, temperature=0.0, stop_token_ids=[], return_stats=True)
            n_dec = stats.steps - 1
            e2e_vals.append(args.batch * n_dec / stats.decode_secs)
            e2e_io = (int((engine.h2d_bytes - h0) / stats.steps), int((engine.d2h_bytes - d0) / stats.steps))
        out["e2e"] = {"value": round(statistics.median(e2e_vals), 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e_io[0],
                      "d2h_bytes_per_step": e2e_io[1], "steps": n_dec, "api": "Engine.generate", "rounds": spread(e2e_vals)}

        times = prefill_point(engine, 2, 1024, iters=max(5, args.rounds), warmup=3, seed=3)
        out["prefill"] = prefill_summary(times, flops_2x1024, 2048, pk, pk_src, args.dtype == "bfloat16")
        points = {}
        sub_steps = min(args.steps, 128)
        for b in (1, 64):
            pt = decode_point(engine, b, args.prompt_len, sub_steps, warmup, seed=10 + b, rounds=args.rounds)
            points[f"decode_b{b}"] = round(pt["tok_s"], 1)
            points[f"decode_b{b}_hbm_frac"] = round(hbm_frac(engine, b, pt, pk), 4)
            points[f"decode_b{b}_rounds"] = pt["tok_s_rounds"]
        if args.batch == 8:
            prompts1 = random_prompts(1, args.prompt_len, engine.vocab_size, seed=5)
            engine.generate(prompts1, max_tokens=4, temperature=0.0, stop_token_ids=[])
            _, stats = engine.generate(prompts1, max_tokens=sub_steps + 1, temperature=0.0, stop_token_ids=[], return_stats=True)
            points["e2e_decode_b1"] = round((stats.steps - 1) / stats.decode_secs, 1)      # the host has the least time per step here
        pt = decode_point(engine, args.batch, args.prompt_len, sub_steps, warmup, seed=30, rounds=args.rounds, sampled=True)
        points[f"decode_b{args.batch}_sampled"] = round(pt["tok_s"], 1)      # temperature 0.7, top-k 40, top-p 0.95
        if args.dtype == "bfloat16":
            e32 = build_engine(model_dir, cfg, "float32", 8 * cfg["n_positions"])
            err = self_check(engine, e32, cfg, seed=6)
            out["checked"] = bool(err < 2e-2)
            out["check"] = {"what": "bfloat16 logits at the ends of two 512-token prompts against the 32-bit engine, same weights",
                            "max_rel_err": round(err, 5), "limit": 2e-2}
            # the 32-bit engine (true 32-bit arithmetic on CUDA cores): decode against the copy bandwidth, prefill as TFLOP/s
            for b in (1, 8):
                pt = decode_point(e32, b, args.prompt_len, min(sub_steps, 64), 3, seed=60 + b, rounds=max(3, args.rounds - 2))
                points[f"fp32_decode_b{b}"] = round(pt["tok_s"], 1)
                points[f"fp32_decode_b{b}_hbm_frac"] = round(hbm_frac(e32, b, pt, pk), 4)
            times = prefill_point(e32, 2, 1024, iters=3, warmup=1, seed=3)
            points["fp32_prefill"] = prefill_summary(times, flops_2x1024, 2048, pk, pk_src, tensor_cores=False)
            e32.cache.book.check_all_free()
            del e32
            torch.cuda.empty_cache()
        out["points"] = points

    from kvad_b200.csrc import build
    out["loaded_libraries"] = [os.path.basename(p) for p in build.loaded_paths()]
    engine.cache.book.check_all_free()
    if args.points == "large":
        del engine
        torch.cuda.empty_cache()
        large_points(out["points"], pk, pk_src, args)
    print(json.dumps(out))
    tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
