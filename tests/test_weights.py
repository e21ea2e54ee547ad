"""Weights: reading by name, the one audit error, dtypes, random-weights mode (no GPU)."""
import json
import os

import numpy as np
import pytest
import torch

from kvad_b200 import write_random_model
from kvad_b200.config import load_config
from kvad_b200.models import Model
from kvad_b200.weights import (Checkpoint, SafetensorsError, WeightSource, WeightsError, collapse,
                               write_safetensors)
from tests.conftest import TINY
from tests.plain.gpt2_plain import read_safetensors


def load(model_dir, dtype=torch.float32):
    arch, cfg = load_config(model_dir)
    model = Model(arch.plan(cfg))
    ckpt = Checkpoint.open_dir(model_dir)
    model.load(WeightSource(ckpt, ignored_suffixes=model.plan.ignored_suffixes), dtype, "cpu")
    return model


def rewrite(model_dir, change):
    path = os.path.join(model_dir, "model.safetensors")
    ckpt = Checkpoint([path])
    tensors = {n: ckpt.read(n) for n in ckpt.names()}
    ckpt.close()
    change(tensors)
    write_safetensors(path, tensors)


def test_roundtrip_and_independent_reader(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "i": torch.arange(6, dtype=torch.int64).view(2, 3)}
    p = str(tmp_path / "x.safetensors")
    write_safetensors(p, t)
    c = Checkpoint([p])
    assert c.names() == ["a", "b", "i"]
    for n in t:
        assert torch.equal(c.read(n), t[n])
    plain = read_safetensors(p)           # the oracle's own reader agrees on the bytes
    assert np.array_equal(plain["a"], t["a"].double().numpy())
    assert np.array_equal(plain["b"], t["b"].double().numpy())


def test_truncated_file_is_refused(tmp_path):
    p = tmp_path / "model.safetensors"
    p.write_bytes(b"\x10\x00")
    with pytest.raises(SafetensorsError):
        Checkpoint([str(p)])
    with pytest.raises(SafetensorsError, match="neither"):
        Checkpoint.open_dir(str(tmp_path / "nowhere"))


def test_loads_and_transposes_conv1d(tmp_path):
    d = str(tmp_path)
    write_random_model(d, TINY["B"], 5)
    m = load(d)
    raw = read_safetensors(os.path.join(d, "model.safetensors"))
    blk = m.blocks[1]
    assert tuple(blk.mixer.qkv.weight.shape) == (3 * 96, 96)                # held [out, in]
    assert np.array_equal(blk.mixer.qkv.weight.double().numpy(), raw["h.1.attn.c_attn.weight"].T)
    assert np.array_equal(blk.mixer.out.weight.double().numpy(), raw["h.1.attn.c_proj.weight"].T)   # square: silent if missed
    assert np.array_equal(blk.feed_forward.down.weight.double().numpy(), raw["h.1.mlp.c_proj.weight"].T)
    assert np.array_equal(m.embedding.weight.double().numpy(), raw["wte.weight"])                   # not transposed
    assert m.param_count() == sum(v.size for v in raw.values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path)
    write_random_model(d, TINY["A"], 5)

    def change(t):
        del t["h.0.ln_1.bias"], t["h.1.ln_1.bias"], t["ln_f.weight"]
        t["h.0.attn.q_norm.weight"] = torch.zeros(4)
        t["wpe.weight"] = torch.zeros(100, 64)
        t["h.1.mlp.c_fc.weight"] = t["h.1.mlp.c_fc.weight"].t().contiguous()     # stored [out,in] by mistake

    rewrite(d, change)
    with pytest.raises(WeightsError) as e:
        load(d)
    msg = str(e.value)
    assert "h.*.ln_1.bias (2 tensors)" in msg and "ln_f.weight" in msg
    assert "h.0.attn.q_norm.weight" in msg
    assert "wpe.weight is [100, 64], the configuration needs [128, 64]" in msg
    assert "h.1.mlp.c_fc.weight is [256, 64], the configuration needs [64, 256]" in msg
    assert sorted(e.value.missing) == ["h.0.ln_1.bias", "h.1.ln_1.bias", "ln_f.weight"]
    assert e.value.unexpected == ["h.0.attn.q_norm.weight"]
    assert len(e.value.wrong_shape) == 2


def test_prefixed_names_and_stored_masks_are_fine(tmp_path):
    d = str(tmp_path)
    write_random_model(d, TINY["A"], 5)

    def change(t):
        for n in list(t):
            t["transformer." + n] = t.pop(n)
        t["transformer.h.0.attn.bias"] = torch.ones(1, 1, 8, 8)            # a stored causal mask is not a weight
        t["transformer.h.0.attn.masked_bias"] = torch.tensor(-1e4)
        t["lm_head.weight"] = torch.zeros(512, 64)                          # tied: ignored by name

    rewrite(d, change)
    load(d)


def test_untied_head(tmp_path):
    d = str(tmp_path)
    write_random_model(d, TINY["C"], 5)
    m = load(d)
    assert m.head.proj.weight is not None and m.head.proj.bias is not None
    assert m.head.proj.weight.data_ptr() != m.embedding.weight.data_ptr()
    rewrite(d, lambda t: t.pop("lm_head.bias"))                              # the bias is optional
    assert load(d).head.proj.bias is None
    rewrite(d, lambda t: t.pop("lm_head.weight"))                            # the matrix is not
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load(d)


def test_dtypes_kept(tmp_path):
    d = str(tmp_path)
    write_random_model(d, TINY["A"], 5)                                      # stored bfloat16
    rewrite(d, lambda t: t.update({"ln_f.weight": t["ln_f.weight"].float() + 1e-4, "ln_f.bias": t["ln_f.bias"].float()}))
    m = load(d, torch.bfloat16)
    assert m.embedding.weight.dtype == torch.bfloat16
    assert m.blocks[0].norm1.gain.dtype == torch.bfloat16
    assert m.head.norm.gain.dtype == torch.float32                           # stored in 32-bit: stays so
    assert float(m.head.norm.gain[0]) != float(m.head.norm.gain[0].to(torch.bfloat16))
    m32 = load(d, torch.float32)
    assert all(t.dtype == torch.float32 for t in m32.tensors())


def test_random_mode_is_seeded(tmp_path):
    a, b, c = str(tmp_path / "a"), str(tmp_path / "b"), str(tmp_path / "c")
    write_random_model(a, TINY["A"], 1)
    write_random_model(b, TINY["A"], 1)
    write_random_model(c, TINY["A"], 2)
    ra, rb, rc = (read_safetensors(os.path.join(x, "model.safetensors")) for x in (a, b, c))
    assert all(np.array_equal(ra[n], rb[n]) for n in ra)
    assert not np.array_equal(ra["wte.weight"], rc["wte.weight"])
    cfg = json.load(open(os.path.join(a, "config.json")))
    assert cfg["model_type"] == "gpt2" and cfg["n_embd"] == 64
    # gains away from 1 and biases away from 0, so a dropped affine shows
    assert abs(ra["h.0.ln_1.weight"].mean() - 1) < 0.05 and ra["h.0.ln_1.weight"].std() > 0.02
    assert ra["h.0.attn.c_attn.bias"].std() > 0.005
    assert ra["h.0.attn.c_proj.weight"].std() < ra["h.0.attn.c_attn.weight"].std()


def test_collapse():
    assert collapse(["h.0.x", "h.1.x", "ln_f.weight"]) == ["h.*.x (2 tensors)", "ln_f.weight"]


@pytest.mark.parametrize("name", ["A32", "B32", "U16"])
def test_folders_the_library_did_not_write(model_dirs, name):
    """Real checkpoint layout from tests/plain/fixture.py: `transformer.` names, Conv1D matrices stored
    [in, out], stored mask buffers, 32-bit or float16 storage, one file or shards behind an index.
    The loader's tensors equal what the plain reader makes of the same files."""
    from tests.conftest import FOREIGN
    from tests.plain.gpt2_plain import read_model_files
    d = model_dirs[name]
    _, stored, shards = FOREIGN[name]
    assert os.path.isfile(os.path.join(d, "model.safetensors")) == (shards == 1)
    assert os.path.isfile(os.path.join(d, "model.safetensors.index.json")) == (shards > 1)
    m = load(d)
    raw, dtypes = read_model_files(d)
    assert set(dtypes.values()) <= {"I64", {"F32": "F32", "F16": "F16"}[stored]}
    blk = m.blocks[1]
    for got, key, transposed in [(blk.mixer.qkv.weight, "attn.c_attn.weight", True), (blk.mixer.out.weight, "attn.c_proj.weight", True),
                                 (blk.feed_forward.up.weight, "mlp.c_fc.weight", True), (blk.feed_forward.down.bias, "mlp.c_proj.bias", False),
                                 (blk.norm2.gain, "ln_2.weight", False)]:
        want = raw["transformer.h.1." + key]
        assert got.dtype == torch.float32
        assert np.array_equal(got.double().numpy(), want.T if transposed else want), key
    assert np.array_equal(m.embedding.weight.double().numpy(), raw["transformer.wte.weight"])      # never transposed
    if name == "U16":
        assert not m.head.tied and np.array_equal(m.head.proj.weight.double().numpy(), raw["lm_head.weight"])
        assert np.array_equal(m.head.proj.bias.double().numpy(), raw["lm_head.bias"])
    if stored == "F32":                     # values that bfloat16 cannot hold: a path that rounded them would show
        w = raw["transformer.h.0.attn.c_attn.weight"]
        from tests.plain.gpt2_plain import round_bf16
        assert np.mean(round_bf16(w) != w) > 0.95
        bf = load(d, torch.bfloat16)
        assert bf.blocks[0].mixer.qkv.weight.dtype == torch.bfloat16 and bf.blocks[0].norm1.gain.dtype == torch.float32
        assert np.array_equal(bf.blocks[0].mixer.qkv.weight.double().numpy(), round_bf16(w).T)
