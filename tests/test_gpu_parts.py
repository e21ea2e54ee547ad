"""Each part alone, outside any model: built by kind from the registries, given weights from a
dict, run on a real step context, and compared with the plain formulas."""
import math

import numpy as np
import pytest
import torch

from kvad_b200 import StepEntry
from kvad_b200.models.plan import LayerCall
from kvad_b200.parts import PartSpec, build_part, part_kinds
from tests.conftest import TINY, random_tokens
from tests.plain.gpt2_plain import PlainGpt2, round_bf16

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
PTOL = {"float32": 3e-6, "bfloat16": 8e-3}


def fetch_from(tensors, dtype):
    def fetch(name, transpose=False, keep_f32=False, optional=False):
        if name not in tensors:
            assert optional, name
            return None
        t = tensors[name]
        t = t if (keep_f32 and t.dtype == torch.float32) else t.to(dtype)
        return (t.t() if transpose else t).contiguous().cuda()
    return fetch


def rel(got, ref):
    got = got.double().cpu().numpy()
    assert np.isfinite(got).all()
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def stored(t, dtype):
    """A tensor as the engine holds it (rounded to the compute dtype), in float64."""
    return t.to(DT[dtype]).double().numpy()


@pytest.fixture
def step(engines):
    """A real step context on tiny model A: two sequences, 70 and 9 rows."""
    def make(dtype):
        e = engines("A", dtype)
        slots = [e.open(), e.open()]
        toks = [random_tokens(1, 70, 512), random_tokens(2, 9, 512)]
        ctx = e.begin_step([StepEntry(s, t, [len(t) - 1]) for s, t in zip(slots, toks)])
        return e, ctx, slots, toks
    made = []

    def get(dtype):
        made.append(make(dtype))
        return made[-1]
    yield get
    for e, ctx, slots, _ in made:
        for s in slots:
            e.close(s)


def test_every_family_has_its_built_in_kinds():
    assert "layernorm" in part_kinds("norm") and "causal_attention" in part_kinds("mixer")
    assert "dense_mlp" in part_kinds("feed_forward") and "pre_norm" in part_kinds("block")
    assert {"learned_absolute", "none"} <= set(part_kinds("position"))
    with pytest.raises(ValueError, match="no mixer of kind"):
        build_part("mixer", PartSpec("does_not_exist", {}))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_alone(step, dtype):
    e, ctx, _, _ = step(dtype)
    g = torch.Generator().manual_seed(1)
    w, b = 1 + 0.1 * torch.randn(64, generator=g), 0.1 * torch.randn(64, generator=g)
    norm = build_part("norm", PartSpec("layernorm", {"width": 64, "eps": 1e-3}), "n.")
    assert [r.name for r in norm.requests()] == ["n.weight", "n.bias"]
    norm.load(fetch_from({"n.weight": w, "n.bias": b}, DT[dtype]))
    x = torch.randn(ctx.n_rows, 64, generator=g) * 2 + 0.5
    out = norm.forward(ctx, x.cuda())
    xd = x.double().numpy()
    mean, var = xd.mean(-1, keepdims=True), xd.var(-1, keepdims=True)
    ref = (xd - mean) / np.sqrt(var + 1e-3) * stored(w, dtype) + stored(b, dtype)
    assert out.dtype == DT[dtype] and rel(out, ref) < PTOL[dtype]
    out = norm.forward(ctx, x.cuda(), rows=ctx.want_rows, n_rows=2)           # only the wanted rows
    assert rel(out, ref[[69, 78]]) < PTOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_embedding_and_positions_alone(step, dtype):
    e, ctx, _, toks = step(dtype)
    g = torch.Generator().manual_seed(2)
    wte, wpe = torch.randn(512, 48, generator=g), torch.randn(128, 48, generator=g)
    emb = build_part("embedding", PartSpec("token_embedding", {
        "vocab_size": 512, "width": 48, "name": "tok.weight",
        "position": PartSpec("learned_absolute", {"n_positions": 128, "width": 48, "name": "pos.weight"})}), "")
    assert emb.max_positions == 128
    emb.load(fetch_from({"tok.weight": wte, "pos.weight": wpe}, DT[dtype]))
    x = emb.forward(ctx)
    ref = np.concatenate([stored(wte, dtype)[t] + stored(wpe, dtype)[: len(t)] for t in toks])
    assert x.dtype == torch.float32 and rel(x, ref) < 1e-7
    bare = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 512, "width": 48, "name": "tok.weight",
                                                                "position": PartSpec("none", {})}), "")
    bare.load(fetch_from({"tok.weight": wte}, DT[dtype]))
    assert bare.max_positions is None
    assert rel(bare.forward(ctx), np.concatenate([stored(wte, dtype)[t] for t in toks])) < 1e-7


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_alone(step, dtype):
    e, ctx, _, _ = step(dtype)
    g = torch.Generator().manual_seed(3)
    for act, fn in (("gelu_tanh", PlainGpt2.gelu_tanh), ("gelu_erf", PlainGpt2.gelu_erf)):
        t = {"ff.up.weight": torch.randn(64, 200, generator=g) * 0.2, "ff.up.bias": torch.randn(200, generator=g) * 0.1,
             "ff.down.weight": torch.randn(200, 64, generator=g) * 0.1, "ff.down.bias": torch.randn(64, generator=g) * 0.1}
        ff = build_part("feed_forward", PartSpec("dense_mlp", {"width": 64, "hidden": 200, "activation": act, "stored": "in_out"}), "ff.")
        ff.load(fetch_from(t, DT[dtype]))
        h = (torch.randn(ctx.n_rows, 64, generator=g)).to(DT[dtype])
        base = torch.randn(ctx.n_rows, 64, generator=g)
        resid = base.clone().cuda()
        ff.forward(ctx, h.cuda(), resid)
        hid = fn(h.double().numpy() @ stored(t["ff.up.weight"], dtype) + stored(t["ff.up.bias"], dtype))
        if dtype == "bfloat16":
            hid = round_bf16(hid)
        ref = base.double().numpy() + hid @ stored(t["ff.down.weight"], dtype) + stored(t["ff.down.bias"], dtype)
        assert rel(resid, ref) < PTOL[dtype], act
    with pytest.raises(ValueError, match="no activation"):
        build_part("feed_forward", PartSpec("dense_mlp", {"width": 8, "hidden": 8, "activation": "relu"}), "")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_mixer_alone(step, dtype, plains):
    """The mixer with weights of its own on the engine's cache entry 0 (4 heads of 16, as tiny A has)."""
    e, ctx, _, toks = step(dtype)
    g = torch.Generator().manual_seed(4)
    t = {"a.qkv.weight": torch.randn(192, 64, generator=g) * 0.3, "a.qkv.bias": torch.randn(192, generator=g) * 0.1,
         "a.out.weight": torch.randn(64, 64, generator=g) * 0.2, "a.out.bias": torch.randn(64, generator=g) * 0.1}
    mixer = build_part("mixer", PartSpec("causal_attention", {"width": 64, "n_heads": 4, "head_dim": 16, "score_scale": 0.3}), "a.")
    assert mixer.cache_need() == e.model.blocks[0].mixer.cache_need()
    mixer.load(fetch_from(t, DT[dtype]))
    h = torch.randn(ctx.n_rows, 64, generator=g).to(DT[dtype])
    resid = torch.zeros(ctx.n_rows, 64).cuda()
    mixer.forward(ctx, h.cuda(), resid, LayerCall(0, 0))
    plain = plains("A")
    rnd = round_bf16 if dtype == "bfloat16" else (lambda a: a)
    ref, off = [], 0
    for tk in toks:
        hh = h[off:off + len(tk)].double().numpy()
        qkv = rnd(hh @ stored(t["a.qkv.weight"], dtype).T + stored(t["a.qkv.bias"], dtype))
        scale_fix = 0.3 * math.sqrt(16)                      # plain.attention scales by 1/sqrt(16); this mixer by 0.3
        a = rnd(plain.attention(qkv[:, :64] * scale_fix, qkv[:, 64:128], qkv[:, 128:], 0))
        ref.append(a @ stored(t["a.out.weight"], dtype).T + stored(t["a.out.bias"], dtype))
        off += len(tk)
    assert rel(resid, np.concatenate(ref)) < PTOL[dtype] * (3 if dtype == "bfloat16" else 1)
    with pytest.raises(ValueError, match="multiple of 16"):
        build_part("mixer", PartSpec("causal_attention", {"width": 8, "n_heads": 1, "head_dim": 8, "score_scale": 1.0}), "")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_head_alone_tied_and_untied(step, dtype):
    e, ctx, _, _ = step(dtype)
    g = torch.Generator().manual_seed(5)
    wte = torch.randn(777, 64, generator=g) * 0.1
    t = {"tok.weight": wte, "f.weight": 1 + 0.1 * torch.randn(64, generator=g), "f.bias": 0.1 * torch.randn(64, generator=g),
         "out.weight": torch.randn(777, 64, generator=g) * 0.1, "out.bias": torch.randn(777, generator=g) * 0.1}
    emb = build_part("embedding", PartSpec("token_embedding", {"vocab_size": 777, "width": 64, "name": "tok.weight"}), "")
    emb.load(fetch_from(t, DT[dtype]))
    x = torch.randn(ctx.n_rows, 64, generator=g)
    xd = x.double().numpy()[[69, 78]]
    normed = (xd - xd.mean(-1, keepdims=True)) / np.sqrt(xd.var(-1, keepdims=True) + 1e-5) * stored(t["f.weight"], dtype) + stored(t["f.bias"], dtype)
    if dtype == "bfloat16":
        normed = round_bf16(normed)
    norm = PartSpec("layernorm", {"width": 64, "eps": 1e-5})
    for tied in (True, False):
        head = build_part("head", PartSpec("lm_head", {"vocab_size": 777, "width": 64, "norm": norm, "tied": tied, "bias": True,
                                                       "norm_name": "f.", "name": "out."}), "", embedding=emb)
        names = [r.name for r in head.requests()]
        assert ("out.weight" in names) == (not tied)
        head.load(fetch_from(t, DT[dtype]))
        logits = head.forward(ctx, x.cuda())
        ref = normed @ (stored(wte, dtype).T if tied else stored(t["out.weight"], dtype).T) + (0 if tied else stored(t["out.bias"], dtype))
        assert logits.dtype == torch.float32 and tuple(logits.shape) == (2, 777)
        assert rel(logits, ref) < PTOL[dtype], tied
        if tied:
            assert head.proj.weight.data_ptr() == emb.weight.data_ptr()           # no second copy of the table


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_block_alone(step, dtype, plains):
    """The pre-norm arrangement built from the plan's own spec with weights of its own names, on rows that are
    no model's activations: x += mixer(norm1(x)); x += feed_forward(norm2(x)), on cache entry 1."""
    e, ctx, _, toks = step(dtype)
    plain = plains("A")
    spec = e.model.plan.blocks[1]
    block = build_part("block", spec, "blk.")
    assert [type(c).__name__ for c in block.children()] == ["LayerNorm", "CausalSelfAttention", "LayerNorm", "DenseMLP"]
    # the part's requests name what it wants; feed it layer 1's tensors of tiny A under those names
    theirs = {r.name: r for r in e.model.blocks[1].requests()}
    mine = {r.name: r for r in block.requests()}
    assert len(theirs) == len(mine) == 12
    rename = {m: t for m, t in zip(sorted(mine), sorted(theirs))}     # same suffixes, other prefix: same order
    assert all(m.split(".", 1)[1] == t.split(".", 2)[2] for m, t in rename.items()), rename
    tensors = {m: torch.from_numpy(np.asarray(plain.w[t])) for m, t in rename.items()}
    block.load(fetch_from(tensors, DT[dtype]))
    g = torch.Generator().manual_seed(11)
    x0 = torch.randn(ctx.n_rows, 64, generator=g)
    x = x0.clone().cuda()
    block.forward(ctx, x, LayerCall(1, 1))
    ref, off = [], 0
    for tk in toks:
        ref.append(plain.block(x0[off:off + len(tk)].double().numpy(), 1))
        off += len(tk)
    assert rel(x, np.concatenate(ref)) < PTOL[dtype] * (3 if dtype == "bfloat16" else 1)
