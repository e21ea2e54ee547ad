"""Command line in bisand/kvad's manner: `kvad run --model DIR --prompt TEXT`.

Option names, meanings and defaults are `kvad run`'s where it has them
(crates/llm/src/cli/spec.rs:1176-1209, crates/llm/src/main.rs:249-252, 315,
crates/llm/src/service.rs:182-191): `--temperature 0.7`, `--top-k 40`,
`--top-p 0.95`, `--seed 7`, `--greedy` for `--temperature 0`, `--max-tokens`
256 for a continuation; `--dtype` is the GPU binary's (crates/gpu/src/main.rs:45-63).
Text goes to standard output, everything else to standard error, and a run ends
with `[prefill N tokens in Xs · generated M in Ys = Z tok/s]`
(crates/llm/src/main.rs:1613-1617).  `kvad arch` lists the registry
(crates/llm/src/main.rs:782-798).

Tokenising is outside the library.  If the model folder has a `tokenizer.json`
and the `tokenizers` package is installed, `--prompt` is encoded and the reply
decoded with it; otherwise give token ids with `--tokens` and ids come back.
`--random-weights CONFIG.json --model DIR` first writes a random model folder.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

DEFAULT_PROMPT = "The first time I saw the sea,"      # crates/llm/src/main.rs:1583-1589


def _say(msg: str) -> None:
    print(msg, file=sys.stderr, flush=True)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="kvad", description="kvad_b200: GPT-2 inference on one B200")
    sub = p.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="continue a prompt")
    run.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    run.add_argument("--prompt", action="append", help="what to continue (may be given several times: one batch)")
    run.add_argument("--tokens", action="append", help="a prompt as comma-separated token ids (instead of --prompt)")
    run.add_argument("--max-tokens", type=int, default=256, help="most tokens to write per prompt")
    run.add_argument("--temperature", type=float, default=0.7, help="0 = greedy")
    run.add_argument("--top-k", type=int, default=40, help="0 = off")
    run.add_argument("--top-p", type=float, default=0.95)
    run.add_argument("--seed", type=int, default=7, help="same seed, same text")
    run.add_argument("--greedy", action="store_true", help="--temperature 0")
    run.add_argument("--dtype", default="bf16", choices=["bf16", "bfloat16", "f32", "float32"])
    run.add_argument("--stop", type=int, action="append", help="a stop token id (default: the model's eos ids)")
    run.add_argument("--random-weights", metavar="CONFIG", help="write random weights for CONFIG (a config.json) into --model first")
    run.add_argument("--cache-tokens", type=int, default=0, help="size of the cache in tokens (default: what the prompts need)")
    info = sub.add_parser("info", help="what a model folder holds")
    info.add_argument("--model", required=True)
    sub.add_parser("arch", help="architectures this build runs")
    return p


def cmd_arch() -> int:
    from . import models  # noqa: F401
    from .config import architectures

    for a in architectures():
        print(f"{a.id:10s} {', '.join(a.model_types):20s} {a.about}")
    return 0


def cmd_info(args) -> int:
    from .config import load_config
    from .models.plan import Model
    from .weights import Checkpoint

    arch, cfg = load_config(args.model)
    model = Model(arch.plan(cfg))
    print(model.plan.summary)
    ckpt = Checkpoint.open_dir(args.model)
    n = sum(int(__import__("numpy").prod(e.shape)) for e in ckpt.entries.values())
    print(f"{len(ckpt.entries)} tensors, {n / 1e6:.2f} M values on disk")
    print(json.dumps(cfg.__dict__, default=str))
    return 0


def cmd_run(args) -> int:
    from .engine.engine import Engine

    if args.random_weights:
        from .weights.random_init import write_random_model
        with open(args.random_weights) as f:
            write_random_model(args.model, json.load(f), args.seed)
        _say(f"wrote random weights to {args.model}")

    tokenizer = None
    tok_path = os.path.join(args.model, "tokenizer.json")
    if os.path.isfile(tok_path):
        try:
            from tokenizers import Tokenizer
            tokenizer = Tokenizer.from_file(tok_path)
        except Exception as e:  # noqa: BLE001
            _say(f"tokenizer.json could not be used ({e}); give --tokens")
    prompts: list[list[int]] = []
    for t in args.tokens or []:
        prompts.append([int(x) for x in t.replace(" ", ",").split(",") if x != ""])
    texts = list(args.prompt or [])
    if not prompts and not texts:
        texts = [DEFAULT_PROMPT]
    if texts:
        if tokenizer is None:
            _say("this model folder has no usable tokenizer.json: give the prompt as --tokens 1,2,3")
            return 2
        prompts.extend(tokenizer.encode(t).ids for t in texts)

    temperature = 0.0 if args.greedy else args.temperature
    t0 = time.time()
    need = sum(-(-(len(p) + args.max_tokens) // 64) * 64 for p in prompts)
    engine = Engine.from_pretrained(args.model, args.dtype, max_tokens=max(args.cache_tokens, need))
    _say(engine.describe())
    _say(f"loaded in {time.time() - t0:.1f} s")
    outs, stats = engine.generate(prompts, max_tokens=args.max_tokens, temperature=temperature, top_k=args.top_k,
                                  top_p=args.top_p, seed=args.seed, stop_token_ids=args.stop, return_stats=True)
    for i, (p, o) in enumerate(zip(prompts, outs)):
        if tokenizer is not None and texts:
            print(tokenizer.decode(list(p) + o))          # a base model's output starts with its prompt
        else:
            print(",".join(str(t) for t in o))
    _say(f"[prefill {stats.prompt_tokens} tokens in {stats.prefill_secs:.2f}s · generated {stats.generated_tokens} in "
         f"{stats.decode_secs:.2f}s = {stats.tokens_per_sec():.1f} tok/s]")
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.command == "arch":
        return cmd_arch()
    if args.command == "info":
        return cmd_info(args)
    return cmd_run(args)
