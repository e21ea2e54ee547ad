"""The engine: a loaded model, its cache, and ONE step function.

`Engine.step(entries)` is everything between a request's tokens and its next
token: it runs exactly the tokens it is given - prompts of unequal lengths in
one step, or one token per sequence - as one packed batch from the cache, and
returns the 32-bit logits at the wanted places.  Generation, trace replay and
the benchmark all call it; there is no second forward pass.

bisand/kvad's counterpart is `Session::forward` / `forward_each`
(crates/llm/src/model/mod.rs:839-976) over `Transformer::{embed, blocks, head}`
(crates/llm/src/model/gpt2.rs:200-287); the Python entry point has no
counterpart there and follows the names of `Llm` (crates/llm/src/runtime.rs).
"""
from __future__ import annotations

import collections
import os
import sys
import tempfile
from typing import Optional, Sequence

import numpy as np
import torch

from ..cache.device import DeviceCache
from ..cache.pages import PAGE_SIZE, CacheError, CacheFull
from ..config import load_config
from ..models.plan import Model
from ..ops import KernelError, Ops, lib, libraries_for
from ..sampling.sampler import SamplingParams
from ..weights.safetensors_io import Checkpoint
from ..weights.source import WeightSource
from .batch import MetaLayout, StepEntry, pack
from .context import Arena, DeviceMeta, StepContext
from .generate import Request, Stats, run_all

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "f32": torch.float32}


def parse_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError("the engine computes in bfloat16 or float32")
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, not `{name}`") from None


class _SampleBuffers:
    """Sampling options of a step's rows (pinned host + device) and the chosen tokens.

    The options go up through a ring of pinned staging buffers, each with an event recorded after
    its copy was queued: a buffer is written again only once the copy that last read it has run.
    The generation loop launches a step ahead of the one it waits for, so without the ring the host
    could overwrite a step's uniform numbers before the device had fetched them."""

    STAGES = 4

    def __init__(self, cap: int, device):
        self._hosts = [torch.zeros((4, cap), dtype=torch.float32).pin_memory() for _ in range(self.STAGES)]
        self._events: list = [None] * self.STAGES
        self._next = 0
        self.cap = cap
        self.dev = torch.zeros((4, cap), dtype=torch.float32, device=device)
        self.out = torch.zeros(cap, dtype=torch.int32, device=device)
        self.out_host = torch.zeros(cap, dtype=torch.int32).pin_memory()
        self.out_hosts = [torch.zeros(cap, dtype=torch.int32).pin_memory() for _ in range(2)]   # for reads that lag a step
        self._parity = 0
        self.scratch = None                    # of the two-stage argmax

    def load(self, samplers, engine) -> bool:
        """Uploads temperature, top-p, this step's uniform draw and top-k per row; True if all rows are greedy."""
        if all(s.params.greedy for s in samplers):
            return True
        i = self._next
        self._next = (i + 1) % self.STAGES
        if self._events[i] is not None:
            self._events[i].synchronize()
        host = self._hosts[i]
        h = host.numpy()
        hk = h[3].view(np.int32)
        for j, s in enumerate(samplers):
            h[0, j] = s.params.temperature
            h[1, j] = s.params.top_p
            h[2, j] = s.next_uniform()
            hk[j] = s.params.top_k
        self.dev.copy_(host, non_blocking=True)
        ev = self._events[i] or torch.cuda.Event()
        ev.record()
        self._events[i] = ev
        engine.h2d_bytes += host.numel() * 4
        return False

    def read_async(self, n: int, engine) -> "_PendingTokens":
        """Starts the copy of the chosen tokens to the host and returns a handle; two host buffers
        alternate, so a step launched ahead does not overwrite what the host has yet to read."""
        host = self.out_hosts[self._parity]
        self._parity ^= 1
        host[:n].copy_(self.out[:n], non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        return _PendingTokens(host, n, event, engine)

    def read(self, n: int, engine) -> list[int]:
        self.out_host[:n].copy_(self.out[:n], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        engine.d2h_bytes += 4 * n
        return self.out_host[:n].tolist()


class _PendingTokens:
    """Chosen tokens of a launched step, on their way to the host."""

    def __init__(self, host: torch.Tensor, n: int, event, engine):
        self.host, self.n, self.event, self.engine = host, n, event, engine

    def tokens(self) -> list[int]:
        self.event.synchronize()
        self.engine.d2h_bytes += 4 * self.n
        return self.host[:self.n].tolist()


class _DecodePlan:
    def __init__(self, meta: DeviceMeta, bufs: _SampleBuffers):
        self.meta, self.bufs = meta, bufs


class Engine:
    def __init__(self, model: Model, config, *, max_tokens: int = 65536, max_seqs: Optional[int] = None,
                 verbose: bool = False):
        if model.dtype is None:
            raise ValueError("the model has no weights yet")
        if model.device.type != "cuda":
            raise KernelError("kvad_b200 runs on a CUDA device; there is no CPU path")
        self.model = model
        self.config = config
        self.dtype = model.dtype
        self.device = model.device
        self.vocab_size = model.plan.vocab_size
        self.max_positions = model.max_positions
        self.ops = Ops(self.dtype)
        self.cache = DeviceCache(model.cache_layout, self.dtype, self.device, max_tokens,
                                 max_seqs=max_seqs, max_positions=self.max_positions, page_size=PAGE_SIZE)
        self.arena = Arena(self.device, 1 << 20)
        self._metas: dict[tuple[int, int], DeviceMeta] = {}
        self._table_widths = {g: self.cache.table_width for g in self.cache.kv_group_ids()}
        self._sample_bufs = None
        self.eos_token_ids = tuple(model.plan.eos_token_ids)
        self.verbose = verbose
        from .. import profile
        # a part that reads host-side step data keeps the model on plain launches; so does the per-operation time table
        self.use_graphs = model.graph_safe and not profile.enabled()
        self.max_graphs = 48            # captured step shapes kept (least recently used go first)
        self._graphs: "collections.OrderedDict" = collections.OrderedDict()
        self._decode_plans: dict = {}
        self.h2d_bytes = 0          # bytes copied host -> device by steps and sampling (for measurement)
        self.d2h_bytes = 0
        self.graph_kernels = 0      # kernels of this library run by decode steps (graph replays count their kernels)

    # -- loading -------------------------------------------------------------------
    @classmethod
    def from_pretrained(cls, model_dir: str, dtype="bfloat16", *, device="cuda:0", max_tokens: int = 65536,
                        max_seqs: Optional[int] = None, verbose: bool = False) -> "Engine":
        """Loads a model folder (config.json + safetensors); the class is chosen by config.json."""
        tdtype = parse_dtype(dtype)
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: kvad_b200 has no CPU path")
        torch.cuda.set_device(torch.device(device))
        # compile (first call only) what this model needs, before the weights take time
        from ..csrc import build
        build.build_all(libraries_for(tdtype), verbose=True)
        arch, config = load_config(model_dir)
        model = Model(arch.plan(config))
        ckpt = Checkpoint.open_dir(model_dir)
        try:
            source = WeightSource(ckpt, ignored_suffixes=model.plan.ignored_suffixes)
            model.load(source, tdtype, device)
        finally:
            ckpt.close()
        gen_cfg = os.path.join(model_dir, "generation_config.json")
        eng = cls(model, config, max_tokens=max_tokens, max_seqs=max_seqs, verbose=verbose)
        if os.path.isfile(gen_cfg):
            from ..config.json_view import JsonView
            extra = JsonView.from_file(gen_cfg).id_list("eos_token_id")
            eng.eos_token_ids = tuple(sorted(set(eng.eos_token_ids) | set(extra)))
        return eng

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", *, model_dir: Optional[str] = None, **kw) -> "Engine":
        """Random weights: writes a model folder from `config` (a dict in config.json's keys, or a
        typed configuration) and `seed`, then loads it like any other."""
        from ..weights.random_init import write_random_model
        if model_dir is None:
            with tempfile.TemporaryDirectory(prefix="kvad_b200-random-") as tmp:
                write_random_model(tmp, config, seed)
                return cls.from_pretrained(tmp, dtype, **kw)
        write_random_model(model_dir, config, seed)
        return cls.from_pretrained(model_dir, dtype, **kw)

    # -- sequences -------------------------------------------------------------------
    def open(self) -> int:
        """A slot for a new sequence."""
        return self.cache.acquire()

    def close(self, slot: int) -> None:
        """Gives back everything the sequence holds."""
        self.cache.release(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    def room(self, prompt_len: int) -> int:
        """How many tokens still fit after a prompt of this length: up to the model's own bound, or,
        for a model without one, up to what the whole cache holds."""
        bound = self.max_positions if self.max_positions is not None else self.cache.max_tokens
        return bound - prompt_len

    # -- the step ----------------------------------------------------------------------
    def _meta_for(self, n_rows: int, n_seqs: int) -> DeviceMeta:
        def bucket(n):
            b = 16
            while b < n:
                b *= 2
            return b
        key = (bucket(n_rows), bucket(n_seqs))
        m = self._metas.get(key)
        if m is None:
            m = DeviceMeta(MetaLayout(key[0], key[1], self._table_widths), self.device)
            self._metas[key] = m
        return m

    def begin_step(self, entries: Sequence[StepEntry], *, meta: Optional[DeviceMeta] = None,
                   keep_tokens: bool = False) -> StepContext:
        """Checks and packs a step, makes room in the cache, uploads the metadata."""
        entries = list(entries)
        for e in entries:
            if not self.cache.book.slots.is_out(e.slot):
                raise CacheError(f"slot {e.slot} is not open")
        firsts = [self.cache.length(e.slot) for e in entries]
        batch = pack(entries, firsts, self.vocab_size)
        grown = []
        try:
            for e in entries:
                self.cache.book.grow(e.slot, len(e.tokens))
                grown.append(e)
        except CacheError:
            for e, first in zip(grown, firsts):
                self.cache.book.truncate(e.slot, first)
            raise
        tables = {g: [self.cache.pages_of(e.slot, g) for e in entries] for g in self.cache.kv_group_ids()}
        meta = meta or self._meta_for(batch.n_rows, batch.n_seqs)
        self.h2d_bytes += meta.upload(batch, tables, keep_tokens=keep_tokens)
        self.arena.reset()
        ctx = StepContext(self.ops, self.cache, self.arena, meta, batch)
        ctx.entries = entries
        return ctx

    def end_step(self, ctx: StepContext) -> None:
        for e in ctx.entries:
            self.cache.book.trim_windows(e.slot)

    def step(self, entries: Sequence[StepEntry]) -> torch.Tensor:
        """Runs the given tokens of the given sequences as one batch.

        Returns float32 logits `[wanted rows, vocab]` in the order of the entries
        and of their `want` lists.  The tensor is scratch: it is valid until the
        next step.  A step that is refused (unknown slot, token outside the
        vocabulary, full context, full cache) changes nothing.

        A step's kernels depend only on its shape (rows, sequences, the longest
        run of new rows, wanted rows), never on positions or lengths, which live
        in device memory.  So the second time a shape is seen its launch sequence
        is captured as a CUDA graph and later steps of that shape replay it: one
        upload and one launch instead of a launch per kernel from the host."""
        ctx = self.begin_step(entries)
        b = ctx.batch
        key = ("step", b.n_rows, b.n_seqs, b.max_new, ctx.n_want, id(ctx.meta), self.arena.generation,
               self.ops.path_key())
        logits = self._replay_or_run(key, lambda: self.model.forward(ctx))
        self.end_step(ctx)
        return logits

    def _replay_or_run(self, key, body):
        """Runs `body` (a sequence of kernel launches on fixed addresses) kernel by kernel the first
        time `key` is seen, captures it the second time, replays it from then on.  Returns what
        `body` returned when it was captured (tensors at fixed addresses)."""
        from .. import ops as ops_mod
        if not self.use_graphs:
            return body()
        hit = self._graphs.get(key)
        if hit is not None and hit != "seen":
            graph, result, n_kernels = hit
            self._graphs.move_to_end(key)
            graph.replay()
            self.graph_kernels += n_kernels
            return result
        if hit is None:
            self._graphs[key] = "seen"
            while len(self._graphs) > self.max_graphs:
                self._graphs.popitem(last=False)
            before = ops_mod.launch_count()
            result = body()
            self.graph_kernels += ops_mod.launch_count() - before
            return result
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = ops_mod.launch_count()
        with torch.cuda.graph(graph):
            result = body()
        n_kernels = ops_mod.launch_count() - before
        self._graphs[key] = (graph, result, n_kernels)
        graph.replay()
        self.graph_kernels += n_kernels
        return result

    # -- sampling on the device ----------------------------------------------------------
    def _sampling_buffers(self, n: int):
        if self._sample_bufs is None or self._sample_bufs.cap < n:
            cap = max(64, 1 << (n - 1).bit_length())
            self._sample_bufs = _SampleBuffers(cap, self.device)
        return self._sample_bufs

    def sample(self, logits: torch.Tensor, samplers) -> list[int]:
        """One token per row of `logits`, by each row's own options and stream."""
        n = logits.shape[0]
        bufs = self._sampling_buffers(n)
        greedy = bufs.load(samplers, self)
        self._run_sampler(logits, bufs, greedy)
        return bufs.read(n, self)

    def _run_sampler(self, logits, bufs, greedy: bool) -> None:
        if greedy:
            n, vocab = logits.shape
            need = n * -(-vocab // self.ops.ARGMAX_CHUNK)
            if bufs.scratch is None or bufs.scratch.numel() < need:
                bufs.scratch = torch.zeros(max(need, bufs.out.numel() * -(-vocab // self.ops.ARGMAX_CHUNK)),
                                           dtype=torch.int64, device=self.device)
            self.ops.argmax(logits, bufs.out, bufs.scratch)
        else:
            d = bufs.dev
            self.ops.sample(logits, d[0], d[3].view(torch.int32), d[1], d[2], bufs.out)

    def step_and_sample(self, entries, samplers) -> list[int]:
        """The generation loop's backend call: last-row logits of each entry, then a token each."""
        if all(len(toks) == 1 for _, toks in entries):
            plan = self._decode(entries, samplers)
            return plan.bufs.read(len(entries), self)
        logits = self.step([StepEntry(slot, toks, (len(toks) - 1,)) for slot, toks in entries])
        return self.sample(logits, samplers)

    def launch_step(self, entries, samplers, device_fed: bool = False) -> _PendingTokens:
        """One token per sequence, launched and not waited for.  `entries`: [(slot, [token])], or
        [(slot, None)] with `device_fed`: the tokens are the ones the step before chose for the same
        sequences in the same order, still on the device.  Returns a handle whose `tokens()` waits."""
        ents = [(slot, toks if toks is not None else [0]) for slot, toks in entries]
        plan = self._decode(ents, samplers, device_fed=device_fed)
        return plan.bufs.read_async(len(ents), self)

    # -- decoding through a captured graph -----------------------------------------------
    def _decode(self, entries, samplers, *, device_fed: bool = False) -> "_DecodePlan":
        """One token per sequence, then a token chosen for each; leaves the chosen tokens on the device
        (in `plan.bufs.out`, and in the token section of the plan's metadata, ready to be the next
        step's input).  Captured and replayed like any other step shape: one upload and one launch."""
        n = len(entries)
        plan = self._decode_plans.get(n)
        if plan is None:
            cap = max(16, 1 << (n - 1).bit_length())
            plan = _DecodePlan(DeviceMeta(MetaLayout(cap, cap, self._table_widths), self.device),
                               _SampleBuffers(cap, self.device))
            self._decode_plans[n] = plan
        ctx = self.begin_step([StepEntry(slot, toks, (0,)) for slot, toks in entries], meta=plan.meta,
                              keep_tokens=device_fed)
        greedy = plan.bufs.load(samplers, self)
        key = ("decode", n, greedy, id(plan.meta), self.arena.generation, self.ops.path_key())
        self._replay_or_run(key, lambda: self._decode_body(ctx, plan, greedy))
        self.end_step(ctx)
        return plan

    def _decode_body(self, ctx, plan, greedy: bool) -> None:
        logits = self.model.forward(ctx)
        self._run_sampler(logits, plan.bufs, greedy)
        plan.meta.tokens[:ctx.n_rows].copy_(plan.bufs.out[:ctx.n_rows])

    def decode_run(self, slots: Sequence[int], first_tokens: Sequence[int], steps: int,
                   samplers=None) -> torch.Tensor:
        """`steps` decode steps of the given sequences back to back, each step's chosen tokens feeding
        the next on the device; the host neither waits nor reads in between.  Returns the chosen
        tokens `[steps, sequences]` (int32, on the device).  Nothing stops a sequence early here;
        generation with stop tokens goes through `generate`."""
        from ..sampling.sampler import RequestSampler
        n = len(slots)
        samplers = samplers or [RequestSampler(SamplingParams.make_greedy()) for _ in slots]
        history = torch.empty((steps, n), dtype=torch.int32, device=self.device)
        for k in range(steps):
            toks = first_tokens if k == 0 else [0] * n
            plan = self._decode([(s, [int(t)]) for s, t in zip(slots, toks)], samplers, device_fed=k > 0)
            history[k].copy_(plan.bufs.out[:n])
        return history

    # -- generation ------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_tokens: int = 256, temperature: float = 0.7,
                 top_k: int = 40, top_p: float = 0.95, seed: int = 7,
                 stop_token_ids: Optional[Sequence[int]] = None, batch_size: Optional[int] = None,
                 return_stats: bool = False):
        """Continues each prompt (token ids in, token ids out).

        Prompts run in batches of `batch_size` (default: all at once), one batch
        after another.  `temperature <= 0` is greedy.  Request i draws from its
        own stream seeded `seed + i`.  A stop token (default: the model's
        `eos_token_id`s) ends its request and is not part of the output."""
        stops = frozenset(self.eos_token_ids if stop_token_ids is None else stop_token_ids)
        reqs = [Request(list(p), max_tokens, SamplingParams(temperature, top_k, top_p, seed + i), stops)
                for i, p in enumerate(prompts)]
        stats = run_all(self, reqs, batch_size or max(1, len(reqs)))
        outs = [r.generated for r in reqs]
        return (outs, stats) if return_stats else outs

    # -- replay ------------------------------------------------------------------------------
    def logits_replay(self, steps, out_dir: str) -> int:
        """Feeds given tokens step by step and writes the wanted logits as `<out_dir>/<step>.f32`;
        nothing is sampled.  `steps`: an iterable of trace records (dicts, or JSON lines) in the format
        of `bin/trace_run`.  Returns the number of steps run."""
        import json as _json

        from .replay import Replayer
        rep = Replayer(self, out_dir)
        n = 0
        for rec in steps:
            if isinstance(rec, (str, bytes)):
                if not rec.strip():
                    continue
                rec = _json.loads(rec)
            rep.run_step(rec)
            n += 1
        rep.close_all()
        return n

    # -- accounting --------------------------------------------------------------------------
    def describe(self) -> str:
        m = self.model
        return (f"{m.plan.summary}\n{m.param_count() / 1e6:.2f} M parameters, "
                f"{m.weight_bytes() / 1e6:.1f} MB of weights in {str(self.dtype).replace('torch.', '')}; "
                f"cache {self.cache.bytes() / 1e6:.1f} MB for {self.cache.max_tokens} tokens "
                f"({self.cache.layout.bytes_per_token(torch.empty((), dtype=self.dtype).element_size())} B per token)")
