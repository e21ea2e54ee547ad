"""The framework's generality, shown with toy parts that live in this test only.

1. A mixer with fixed-size state of its own (a decaying running sum per sequence) is registered,
   put into a toy architecture next to an ordinary attention layer, built through the registries
   from a model folder this test writes, and stepped - whole prompts, token by token, unequal
   batches, a reused slot - without a change to any file of the package.
2. A run order that names a block twice and lets a call read the keys and values another call wrote.

The toy parts compute with torch operators: they are test fixtures, not kernels of the library -
except the toy rotary encoding, which brings a CUDA kernel of its own (tests/kernels/toy_rotary.cu)
through `ops.register_kernels`, the door a real part with its own kernel would use.
"""
import json
import math
import os

import numpy as np
import pytest
import torch

from kvad_b200 import Engine, StepEntry
from kvad_b200.cache import StateNeed
from kvad_b200.config import Architecture, register, unregister
from kvad_b200.models.plan import LayerCall, ModelPlan
from kvad_b200.parts import Linear, Mixer, PartSpec, register_part, unregister_part
from kvad_b200.weights import TensorRequest, write_safetensors
from tests.conftest import random_tokens, rel_err

pytestmark = pytest.mark.gpu
W, V, HID, DECAY = 32, 97, 48, 0.75


class RunningSumMixer(Mixer):
    """state <- decay * state + h_t ;  out_t = state . Wo   (one state vector per sequence)."""

    def __init__(self, prefix, width, decay):
        super().__init__(prefix)
        self.width, self.decay = width, decay
        self.out = Linear(prefix + "wo.", width, width, bias=False)

    def children(self):
        return [self.out]

    def cache_need(self):
        return StateNeed((self.width,), torch.float32)

    def forward(self, ctx, h, residual, call):
        state = ctx.state(call.cache)                      # [slots, width], zeroed when a slot is handed out
        starts, slots = ctx.batch.seq_starts, ctx.batch.seq_slots
        mixed = torch.empty((ctx.n_rows, self.width), dtype=torch.float32, device=h.device)
        for s in range(ctx.n_seqs):                        # rows of a sequence in order
            st = state[int(slots[s])]
            for r in range(int(starts[s]), int(starts[s + 1])):
                st.mul_(self.decay).add_(h[r].float())
                mixed[r] = st
        residual.add_(mixed @ self.out.weight.float().t())


def toy_plan(cfg):
    norm = PartSpec("layernorm", {"width": W, "eps": 1e-5})
    ff = PartSpec("dense_mlp", {"width": W, "hidden": HID, "activation": "gelu_tanh"})
    toy = PartSpec("running_sum", {"width": W, "decay": DECAY})
    att = PartSpec("causal_attention", {"width": W, "n_heads": 2, "head_dim": 16, "score_scale": 0.25})
    blocks = [PartSpec("pre_norm", {"norm1": norm, "mixer": m, "norm2": norm, "feed_forward": ff}) for m in (toy, att, toy)]
    return ModelPlan(arch_id="toy_recurrent", vocab_size=V, width=W,
                     embedding=PartSpec("token_embedding", {"vocab_size": V, "width": W, "name": "emb.weight"}),
                     blocks=tuple(blocks), block_prefixes=("l0.", "l1.", "l2."),
                     head=PartSpec("lm_head", {"vocab_size": V, "width": W, "norm": norm, "tied": True, "norm_name": "fin."}),
                     order=ModelPlan.straight_order(3), summary="toy")


def toy_tensors(seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, std=0.3: torch.randn(*s, generator=g) * std
    t = {"emb.weight": r(V, W, std=1.0), "fin.weight": 1 + r(W, std=0.1), "fin.bias": r(W, std=0.1)}
    for i in range(3):
        p = f"l{i}."
        for n in ("norm1.", "norm2."):
            t[p + n + "weight"], t[p + n + "bias"] = 1 + r(W, std=0.1), r(W, std=0.1)
        t[p + "ff.up.weight"], t[p + "ff.up.bias"] = r(HID, W), r(HID, std=0.1)
        t[p + "ff.down.weight"], t[p + "ff.down.bias"] = r(W, HID), r(W, std=0.1)
        if i == 1:
            t[p + "mixer.qkv.weight"], t[p + "mixer.qkv.bias"] = r(3 * W, W), r(3 * W, std=0.1)
            t[p + "mixer.out.weight"], t[p + "mixer.out.bias"] = r(W, W), r(W, std=0.1)
        else:
            t[p + "mixer.wo.weight"] = r(W, W)
    return t


def toy_plain(t, tokens):
    """The toy model on one whole sequence, float64, straight from the definitions."""
    d = {k: v.double().numpy() for k, v in t.items()}
    ln = lambda x, p: (x - x.mean(-1, keepdims=True)) / np.sqrt(x.var(-1, keepdims=True) + 1e-5) * d[p + "weight"] + d[p + "bias"]
    gelu = lambda v: 0.5 * v * (1 + np.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))
    x = d["emb.weight"][np.asarray(tokens)]
    n = len(tokens)
    for i in range(3):
        p = f"l{i}."
        h = ln(x, p + "norm1.")
        if i == 1:
            qkv = h @ d[p + "mixer.qkv.weight"].T + d[p + "mixer.qkv.bias"]
            out = np.zeros((n, W))
            for hd in range(2):
                q, k, v = (qkv[:, j * W + hd * 16: j * W + hd * 16 + 16] for j in range(3))
                s = np.where(np.tril(np.ones((n, n), bool)), q @ k.T * 0.25, -np.inf)
                pr = np.exp(s - s.max(-1, keepdims=True))
                out[:, hd * 16:hd * 16 + 16] = pr / pr.sum(-1, keepdims=True) @ v
            x = x + out @ d[p + "mixer.out.weight"].T + d[p + "mixer.out.bias"]
        else:
            st, mixed = np.zeros(W), np.zeros((n, W))
            for r in range(n):
                st = DECAY * st + h[r]
                mixed[r] = st
            x = x + mixed @ d[p + "mixer.wo.weight"].T
        h = ln(x, p + "norm2.")
        x = x + gelu(h @ d[p + "ff.up.weight"].T + d[p + "ff.up.bias"]) @ d[p + "ff.down.weight"].T + d[p + "ff.down.bias"]
    return ln(x, "fin.") @ d["emb.weight"].T


@pytest.fixture
def toy_dir(tmp_path):
    register_part("mixer", "running_sum", RunningSumMixer)
    register(Architecture("toy_recurrent", ("toy_recurrent",), "a toy with a stateful mixer", lambda view: dict(view.tree), toy_plan))
    tensors = toy_tensors(5)
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    (tmp_path / "config.json").write_text(json.dumps({"model_type": "toy_recurrent"}))
    yield str(tmp_path), tensors
    unregister("toy_recurrent")
    unregister_part("mixer", "running_sum")


def test_toy_mixer_with_state_is_registered_built_and_stepped(toy_dir):
    d, tensors = toy_dir
    e = Engine.from_pretrained(d, "float32", max_tokens=1024)
    assert not e.use_graphs         # the toy mixer walks host-side step data, so its model is never captured as a graph
    layout = e.model.cache_layout
    assert len(layout.groups) == 2 and len(layout.state_groups) == 1 and len(layout.kv_groups) == 1
    assert [g.entries for g in layout.groups] == [(0, 2), (1,)]           # the two toy layers share a group of their own
    a, b = random_tokens(1, 90, V), random_tokens(2, 23, V)
    ra, rb = toy_plain(tensors, a), toy_plain(tensors, b)
    # whole
    s = e.open()
    assert rel_err(e.step([StepEntry(s, a, range(90))]).cpu().numpy(), ra) < 1e-5
    e.close(s)
    # the same slot again: its state was zeroed, so a fresh sequence does not see the old one's sum
    s2 = e.open()
    assert s2 == s
    assert rel_err(e.step([StepEntry(s2, b, range(23))]).cpu().numpy(), rb) < 1e-5
    e.close(s2)
    # prompts of unequal length in one step, then token by token: the state carries over between steps
    sa, sb = e.open(), e.open()
    got = e.step([StepEntry(sa, a[:60], [59]), StepEntry(sb, b[:5], [4])]).cpu().numpy()
    assert rel_err(got[0], ra[59]) < 1e-5 and rel_err(got[1], rb[4]) < 1e-5
    for j in range(18):
        got = e.step([StepEntry(sa, [a[60 + j]], [0]), StepEntry(sb, [b[5 + j]], [0])]).cpu().numpy()
        assert rel_err(got[0], ra[60 + j]) < 1e-5 and rel_err(got[1], rb[5 + j]) < 1e-5, j
    e.close(sb)                                                                 # b ends earlier
    for j in range(18, 30):
        got = e.step([StepEntry(sa, [a[60 + j]], [0])]).cpu().numpy()
        assert rel_err(got[0], ra[60 + j]) < 1e-5, j
    e.close(sa)
    e.cache.book.check_all_free()
    # and generation through the entry point runs on it too
    outs = e.generate([a[:7], b[:3]], max_tokens=5, temperature=0.0)
    want = []
    for p in (a[:7], b[:3]):
        ids = list(p)
        for _ in range(5):
            ids.append(int(np.argmax(toy_plain(tensors, ids)[-1])))
        want.append(ids[len(p):])
    assert outs == want


def test_toy_runs_in_bfloat16_too(toy_dir):
    d, tensors = toy_dir
    e = Engine.from_pretrained(d, "bfloat16", max_tokens=256)
    rounded = {k: v.bfloat16().float() for k, v in tensors.items()}
    a = random_tokens(3, 40, V)
    s = e.open()
    got = e.step([StepEntry(s, a, range(40))]).cpu().numpy()
    e.close(s)
    assert rel_err(got, toy_plain(rounded, a)) < 3e-2          # bfloat16 activations against a float64 oracle


def test_run_order_names_a_block_twice_and_shares_a_cache(model_dirs, plains):
    """GPT-2's own parts under another order: block 0, block 1, block 1 again (a cache entry of its own),
    then block 0 reading the keys and values its first call wrote."""
    from kvad_b200.models import gpt2
    from kvad_b200.config import JsonView
    from tests.conftest import TINY

    def plan(view_cfg):
        base = gpt2.plan(view_cfg)
        order = (LayerCall(0, 0), LayerCall(1, 1), LayerCall(1, 2), LayerCall(0, 0, writes_cache=False))
        return ModelPlan(**{**base.__dict__, "arch_id": "gpt2_loop", "order": order})

    register(Architecture("gpt2_loop", ("gpt2_loop",), "gpt2 parts, looped order", gpt2.read_config, plan))
    try:
        import shutil, tempfile
        with tempfile.TemporaryDirectory() as d:
            shutil.copy(os.path.join(model_dirs["A"], "model.safetensors"), d)
            cfg = dict(TINY["A"], model_type="gpt2_loop")
            json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
            e = Engine.from_pretrained(d, "float32", max_tokens=512)
        assert len(e.model.cache_layout.needs) == 3
        plain = plains("A")
        t = random_tokens(9, 80, 512)

        def reference(tokens):
            w, x = plain.w, plain.embed(tokens)
            x = plain.block(x, 0)
            x = plain.block(x, 1)
            x = plain.block(x, 1)
            # block 0 again, with the keys and values of its FIRST call (computed from the embedding)
            h0 = plain.layer_norm(plain.embed(tokens), w["h.0.ln_1.weight"], w["h.0.ln_1.bias"])
            kv0 = plain.linear(h0, w["h.0.attn.c_attn.weight"], w["h.0.attn.c_attn.bias"])
            h = plain.layer_norm(x, w["h.0.ln_1.weight"], w["h.0.ln_1.bias"])
            q = plain.linear(h, w["h.0.attn.c_attn.weight"], w["h.0.attn.c_attn.bias"])[:, :64]
            a = plain.attention(q, kv0[:, 64:128], kv0[:, 128:], 0)
            x = x + plain.linear(a, w["h.0.attn.c_proj.weight"], w["h.0.attn.c_proj.bias"])
            h = plain.layer_norm(x, w["h.0.ln_2.weight"], w["h.0.ln_2.bias"])
            x = x + plain.linear(plain.gelu_tanh(plain.linear(h, w["h.0.mlp.c_fc.weight"], w["h.0.mlp.c_fc.bias"])),
                                 w["h.0.mlp.c_proj.weight"], w["h.0.mlp.c_proj.bias"])
            return plain.head(x)

        ref = reference(t)
        s = e.open()
        got = [e.step([StepEntry(s, t[:70], range(70))]).cpu().numpy()]
        for j in range(70, 80):
            got.append(e.step([StepEntry(s, [t[j]], [0])]).cpu().numpy())
        e.close(s)
        assert rel_err(np.concatenate(got), ref) < 5e-6
    finally:
        unregister("gpt2_loop")
    with pytest.raises(ValueError, match="before any call has written"):
        from kvad_b200.models.plan import Model
        base = gpt2.plan(gpt2.read_config(JsonView(TINY["A"])))
        Model(ModelPlan(**{**base.__dict__, "order": (LayerCall(0, 0, writes_cache=False),)}))


def test_layers_with_a_window_have_storage_of_their_own(model_dirs, plains):
    """GPT-2's parts again, but every second layer sees only its latest 40 positions: two groups of cache
    entries with storage of their own, pages of the windowed group handed back as they slide out of reach,
    and the same logits as the plain implementation with the same windows - whole, token by token, and
    with a prompt that continues cached positions."""
    from kvad_b200.models import gpt2
    from tests.conftest import TINY
    WINDOW = 40

    def plan(cfg):
        base = gpt2.plan(cfg)
        blocks = []
        for i, b in enumerate(base.blocks):
            if i % 2 == 0:
                mixer = b.params["mixer"].with_params(window=WINDOW)
                b = PartSpec(b.kind, {**b.params, "mixer": mixer})
            blocks.append(b)
        return ModelPlan(**{**base.__dict__, "arch_id": "gpt2_windowed", "blocks": tuple(blocks)})

    register(Architecture("gpt2_windowed", ("gpt2_windowed",), "gpt2 parts, windows on even layers", gpt2.read_config, plan))
    try:
        import shutil, tempfile
        for dtype in ("float32", "bfloat16"):
            with tempfile.TemporaryDirectory() as d:
                shutil.copy(os.path.join(model_dirs["B"], "model.safetensors"), d)
                json.dump(dict(TINY["B"], model_type="gpt2_windowed"), open(os.path.join(d, "config.json"), "w"))
                e = Engine.from_pretrained(d, dtype, max_tokens=1024)
            layout = e.model.cache_layout
            assert [g.entries for g in layout.groups] == [(0, 2), (1,)] and layout.groups[0].need.window == WINDOW
            plain = plains("B", dtype)

            def reference(tokens):
                x = plain.embed(tokens)
                for i in range(3):
                    x = plain.block(x, i, window=WINDOW if i % 2 == 0 else None)
                return plain.head(x)

            tol = 5e-6 if dtype == "float32" else 8e-3
            t = random_tokens(31, 230, 1000)
            ref = reference(t)
            s = e.open()
            got = [e.step([StepEntry(s, t[:100], range(100))]).cpu().numpy(),
                   e.step([StepEntry(s, t[100:190], range(90))]).cpu().numpy()]       # continues cached positions
            for j in range(190, 230):
                got.append(e.step([StepEntry(s, [t[j]], [0])]).cpu().numpy())
            assert rel_err(np.concatenate(got), ref) < tol, dtype
            # the windowed group has dropped the pages no later row can reach; the other group keeps all
            windowed, full = e.cache.pages_of(s, 0), e.cache.pages_of(s, 1)
            assert [p >= 0 for p in windowed] == [False, False, True, True] and all(p >= 0 for p in full)
            e.close(s)
            e.cache.book.check_all_free()
    finally:
        unregister("gpt2_windowed")


def test_a_position_encoding_that_acts_inside_the_mixer(model_dirs, plains):
    """A toy rotary encoding registered from here: no table at the embedding, queries and keys turned by their
    rows' positions before the keys are cached.  The attention mixer calls `rotate`; nothing else changes."""
    from kvad_b200.models import gpt2
    from kvad_b200.parts import PositionEncoding
    from tests.conftest import TINY
    HD, THETA = 16, 100.0

    def angles(positions):
        inv = THETA ** (-np.arange(0, HD, 2) / HD)
        return np.asarray(positions, dtype=np.float64)[:, None] * inv[None, :]

    from ctypes import c_double, c_int, c_int64, c_void_p
    from kvad_b200 import ops as kops
    kops.register_kernels("toy_rotary", os.path.join(os.path.dirname(__file__), "kernels", "toy_rotary.cu"),
                          {"toy_rotary": [c_int, c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_double, c_void_p]})

    class Rotary(PositionEncoding):
        graph_safe = True              # its kernel reads the rows' positions from device memory

        def __init__(self, prefix, head_dim):
            super().__init__(prefix)
            self.head_dim = head_dim

        def rotate(self, ctx, q, k):
            h = kops.lib("toy_rotary")
            for t in (q, k):
                assert t.stride(1) == 1 and t.shape[1] % self.head_dim == 0
                kops.launch(h, h.toy_rotary(ctx.ops.code, c_void_p(t.data_ptr()), t.stride(0), c_void_p(ctx.row_pos.data_ptr()),
                                            ctx.n_rows, t.shape[1] // self.head_dim, self.head_dim, THETA, kops.stream_ptr()))

    def plan(cfg):
        base = gpt2.plan(cfg)
        blocks = [PartSpec(b.kind, {**b.params, "mixer": b.params["mixer"].with_params(position=PartSpec("toy_rotary", {"head_dim": HD}))})
                  for b in base.blocks]
        emb = PartSpec("token_embedding", {**base.embedding.params, "position": PartSpec("none", {})})
        # no position table bounds this model; the plan states the range the encoding is meant for
        return ModelPlan(**{**base.__dict__, "arch_id": "gpt2_rotary", "blocks": tuple(blocks), "embedding": emb,
                            "max_positions": 300})

    register_part("position", "toy_rotary", Rotary)
    register(Architecture("gpt2_rotary", ("gpt2_rotary",), "gpt2 parts, toy rotary positions", gpt2.read_config, plan))
    try:
        import shutil, tempfile
        with tempfile.TemporaryDirectory() as d:
            shutil.copy(os.path.join(model_dirs["A"], "model.safetensors"), d)
            json.dump(dict(TINY["A"], model_type="gpt2_rotary"), open(os.path.join(d, "config.json"), "w"))
            from kvad_b200.weights import Checkpoint
            ck = Checkpoint([os.path.join(d, "model.safetensors")])
            tensors = {n: ck.read(n) for n in ck.names() if n != "wpe.weight"}      # no position table in this model
            ck.close()
            write_safetensors(os.path.join(d, "model.safetensors"), tensors)
            e = Engine.from_pretrained(d, "float32", max_tokens=512)
        assert e.max_positions == 300 and e.room(100) == 200 and e.cache.table_width == 5
        assert e.use_graphs                     # every part, the toy one included, launches by shape only
        plain = plains("A")

        def reference(tokens):
            ang = angles(range(len(tokens)))
            cos, sin = np.cos(ang), np.sin(ang)

            def rot(q, k):
                out = []
                for t in (q, k):
                    v = t.reshape(t.shape[0], -1, HD // 2, 2).copy()
                    a, b = v[..., 0].copy(), v[..., 1].copy()
                    v[..., 0] = a * cos[:, None, :] - b * sin[:, None, :]
                    v[..., 1] = a * sin[:, None, :] + b * cos[:, None, :]
                    out.append(v.reshape(t.shape[0], -1))
                return out
            x = plain.w["wte.weight"][np.asarray(tokens)]
            for i in range(2):
                x = plain.block(x, i, rotate=rot)
            return plain.head(x)

        t = random_tokens(41, 150, 512)                    # beyond the 128 positions the learned table had
        ref = reference(t)
        before = kops.launch_count()
        s = e.open()
        got = [e.step([StepEntry(s, t[:140], range(140))]).cpu().numpy()]
        for j in range(140, 150):                          # the third and later single-token steps replay a captured graph
            got.append(e.step([StepEntry(s, [t[j]], [0])]).cpu().numpy())
        assert rel_err(np.concatenate(got), ref) < 1e-5
        assert kops.launch_count() > before and any("toy_rotary" in p for p in __import__("kvad_b200.csrc.build", fromlist=["x"]).loaded_paths())
        with pytest.raises(Exception, match="context window of 300"):
            e.step([StepEntry(s, random_tokens(42, 151, 512), [0])])
        e.close(s)
        e.cache.book.check_all_free()
    finally:
        unregister("gpt2_rotary")
        unregister_part("position", "toy_rotary")


def test_a_feed_forward_with_routing(model_dirs, plains):
    """A toy feed-forward with two experts and a router, registered from here: every row goes to the expert
    its 32-bit router logit prefers, the expert's output is scaled by the router's probability.  It replaces
    the dense MLP in one of the two layers; mixers, norms, cache and the step function are untouched."""
    from kvad_b200.models import gpt2
    from kvad_b200.parts import FeedForward
    from tests.conftest import TINY
    E, HID = 64, 48

    class RoutedFF(FeedForward):
        def __init__(self, prefix, width, hidden, n_experts):
            super().__init__(prefix)
            self.width, self.hidden, self.n = width, hidden, n_experts
            self.router = Linear(prefix + "router.", width, n_experts, bias=False)
            self.up = [Linear(f"{prefix}experts.{i}.up.", width, hidden) for i in range(n_experts)]
            self.down = [Linear(f"{prefix}experts.{i}.down.", hidden, width) for i in range(n_experts)]

        def children(self):
            return [self.router, *self.up, *self.down]

        def forward(self, ctx, h, residual):
            hf = h.float()
            logits = hf @ self.router.weight.float().t()                       # router logits in 32-bit
            prob, pick = torch.softmax(logits, -1).max(-1)
            for i in range(self.n):
                rows = (pick == i).nonzero().flatten()
                if rows.numel():
                    hid = torch.nn.functional.gelu(hf[rows] @ self.up[i].weight.float().t() + self.up[i].bias.float(), approximate="tanh")
                    out = hid @ self.down[i].weight.float().t() + self.down[i].bias.float()
                    residual.index_add_(0, rows, out * prob[rows, None])

    def plan(cfg):
        base = gpt2.plan(cfg)
        routed = PartSpec("toy_routed", {"width": E, "hidden": HID, "n_experts": 2})
        blocks = [base.blocks[0], PartSpec("pre_norm", {**base.blocks[1].params, "feed_forward": routed})]
        return ModelPlan(**{**base.__dict__, "arch_id": "gpt2_routed", "blocks": tuple(blocks)})

    register_part("feed_forward", "toy_routed", RoutedFF)
    register(Architecture("gpt2_routed", ("gpt2_routed",), "gpt2 parts, a routed feed-forward in layer 1", gpt2.read_config, plan))
    try:
        import tempfile
        from kvad_b200.weights import Checkpoint
        g = torch.Generator().manual_seed(3)
        with tempfile.TemporaryDirectory() as d:
            ck = Checkpoint([os.path.join(model_dirs["A"], "model.safetensors")])
            tensors = {n: ck.read(n).float() for n in ck.names() if not n.startswith("h.1.mlp.c_")}
            ck.close()
            extra = {"h.1.mlp.router.weight": torch.randn(2, E, generator=g)}
            for i in range(2):
                extra[f"h.1.mlp.experts.{i}.up.weight"] = torch.randn(HID, E, generator=g) * 0.2
                extra[f"h.1.mlp.experts.{i}.up.bias"] = torch.randn(HID, generator=g) * 0.1
                extra[f"h.1.mlp.experts.{i}.down.weight"] = torch.randn(E, HID, generator=g) * 0.2
                extra[f"h.1.mlp.experts.{i}.down.bias"] = torch.randn(E, generator=g) * 0.1
            write_safetensors(os.path.join(d, "model.safetensors"), {**tensors, **extra})
            json.dump(dict(TINY["A"], model_type="gpt2_routed"), open(os.path.join(d, "config.json"), "w"))
            e = Engine.from_pretrained(d, "float32", max_tokens=512)
        plain = plains("A")
        x64 = {k: v.double().numpy() for k, v in extra.items()}

        def reference(tokens):
            w = plain.w
            x = plain.block(plain.embed(tokens), 0)
            # layer 1: GPT-2's attention half, then the routed feed-forward
            h = plain.layer_norm(x, w["h.1.ln_1.weight"], w["h.1.ln_1.bias"])
            qkv = plain.linear(h, w["h.1.attn.c_attn.weight"], w["h.1.attn.c_attn.bias"])
            a = plain.attention(qkv[:, :64], qkv[:, 64:128], qkv[:, 128:], 1)
            x = x + plain.linear(a, w["h.1.attn.c_proj.weight"], w["h.1.attn.c_proj.bias"])
            h = plain.layer_norm(x, w["h.1.ln_2.weight"], w["h.1.ln_2.bias"])
            logits = h @ x64["h.1.mlp.router.weight"].T
            p = np.exp(logits - logits.max(-1, keepdims=True))
            p /= p.sum(-1, keepdims=True)
            pick = p.argmax(-1)
            for r in range(len(tokens)):
                i = pick[r]
                hid = plain.gelu_tanh(h[r] @ x64[f"h.1.mlp.experts.{i}.up.weight"].T + x64[f"h.1.mlp.experts.{i}.up.bias"])
                x[r] = x[r] + (hid @ x64[f"h.1.mlp.experts.{i}.down.weight"].T + x64[f"h.1.mlp.experts.{i}.down.bias"]) * p[r, i]
            return plain.head(x)

        t = random_tokens(51, 60, 512)
        ref = reference(t)
        s = e.open()
        got = [e.step([StepEntry(s, t[:50], range(50))]).cpu().numpy()]
        for j in range(50, 60):
            got.append(e.step([StepEntry(s, [t[j]], [0])]).cpu().numpy())
        e.close(s)
        assert rel_err(np.concatenate(got), ref) < 1e-5
    finally:
        unregister("gpt2_routed")
        unregister_part("feed_forward", "toy_routed")
