"""The engine at the layer sizes of the larger GPT-2s (few layers, small vocabulary, random weights):
widths that are no power of two (1600 = 25 heads of 64; 6400), where the kernels take other roads than
at the tiny test sizes (LayerNorm over more than 1024 columns, 25 K blocks, tiles with ragged edges)."""
import numpy as np
import pytest

from kvad_b200 import Engine, StepEntry, write_random_model
from tests.conftest import TOL, random_tokens, rel_err
from tests.plain.gpt2_plain import PlainGpt2

pytestmark = pytest.mark.gpu

SHAPES = {
    "xl": dict(model_type="gpt2", n_layer=2, n_embd=1600, n_head=25, n_inner=6400, vocab_size=3001, n_positions=512,
               layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "medium": dict(model_type="gpt2", n_layer=2, n_embd=1024, n_head=16, n_inner=4096, vocab_size=2000, n_positions=512,
                   layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    # four heads of 128 over two key/value heads: the tcgen05 prompt attention at its other head size, grouped
    "heads128": dict(model_type="gpt2", n_layer=2, n_embd=512, n_head=4, num_key_value_heads=2, head_dim=128, n_inner=1024,
                     vocab_size=1500, n_positions=512, layer_norm_epsilon=1e-5, activation_function="gelu_new"),
}


@pytest.mark.parametrize("name", ["xl", "medium", "heads128"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_large_layer_sizes(tmp_path, name, dtype):
    cfg = SHAPES[name]
    d = str(tmp_path)
    write_random_model(d, cfg, 77)
    plain = PlainGpt2(d, round_to="bfloat16" if dtype == "bfloat16" else None)
    e = Engine.from_pretrained(d, dtype, max_tokens=2048)
    V = cfg["vocab_size"]
    a, b = random_tokens(1, 200, V), random_tokens(2, 70, V)
    ra, rb = plain.logits(a), plain.logits(b)
    sa, sb = e.open(), e.open()
    got = e.step([StepEntry(sa, a[:190], [0, 100, 189]), StepEntry(sb, b[:65], [64])]).cpu().numpy()
    assert rel_err(got[:3], ra[[0, 100, 189]]) < TOL[dtype] and rel_err(got[3], rb[64]) < TOL[dtype]
    for j in range(5):
        got = e.step([StepEntry(sa, [a[190 + j]], [0]), StepEntry(sb, [b[65 + j]], [0])]).cpu().numpy()
        assert rel_err(got[0], ra[190 + j]) < TOL[dtype], j
        assert rel_err(got[1], rb[65 + j]) < TOL[dtype], j
    e.close(sa), e.close(sb)
    e.cache.book.check_all_free()
