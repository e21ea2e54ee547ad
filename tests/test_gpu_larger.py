"""The engine at GPT-2 medium's and GPT-2 XL's layer sizes - width 1024 / 1600, 16 / 25 heads of 64, inner width
4096 / 6400, vocabulary 50257, 1024 positions - with 2 of their 24 / 48 layers, against the plain implementation,
in 32-bit and in bfloat16.  XL's sizes take forms of the kernels that smaller models never reach: LayerNorm with several warps a row, products whose K
is split in 7 and 25, the q/k/v product that leaves 32-bit sums for the attention kernel to finish (3..16 rows),
the head streamed through registers (one row).  The batch below shrinks from 5 rows to 1, so every one of them
runs; every step shape runs kernel by kernel first and as a replayed graph afterwards.  The cache is NaN-poisoned."""
import numpy as np
import pytest

from kvad_b200 import Engine, StepEntry, write_random_model
from tests.conftest import TOL, random_tokens, rel_err
from tests.plain.gpt2_plain import PlainGpt2

pytestmark = pytest.mark.gpu

SIZES = {        # 2 layers of each run here
    "medium": dict(model_type="gpt2", n_layer=2, n_embd=1024, n_head=16, n_inner=4096, vocab_size=50257, n_positions=1024,
                   layer_norm_epsilon=1e-5, activation_function="gelu_new"),
    "xl": dict(model_type="gpt2", n_layer=2, n_embd=1600, n_head=25, n_inner=6400, vocab_size=50257, n_positions=1024,
               layer_norm_epsilon=1e-5, activation_function="gelu_new"),
}
V = 50257


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = str(tmp_path_factory.mktemp("gpt2" + name))
            write_random_model(made[name], SIZES[name], seed=61)
        return made[name]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["medium", "xl"])
def test_unequal_batch_that_shrinks_to_one_row(model_dir, name, dtype):
    xl_dir = model_dir(name)
    e = Engine.from_pretrained(xl_dir, dtype, max_tokens=4096)
    for k, v in e.cache.kv.values():
        k.fill_(float("nan"))
        v.fill_(float("nan"))
    plain = PlainGpt2(xl_dir, round_to="bfloat16" if dtype == "bfloat16" else None)
    prompt_lens = [70, 1, 64, 33, 130]
    extra = [12, 10, 7, 5, 3]                       # decoded tokens: 5 rows for 3 steps, then 4, 3, 2 and 1
    seqs = [random_tokens(1500 + i, p + x, V) for i, (p, x) in enumerate(zip(prompt_lens, extra))]
    refs = [plain.logits(t, rows=range(p - 1, len(t))) for t, p in zip(seqs, prompt_lens)]
    slots = [e.open() for _ in seqs]
    got = e.step([StepEntry(s, t[:p], [p - 1]) for s, t, p in zip(slots, seqs, prompt_lens)]).cpu().numpy()
    for i in range(len(seqs)):
        assert rel_err(got[i], refs[i][0]) < TOL[dtype], f"end of prompt {i} ({prompt_lens[i]} tokens)"
    live, step, sizes = list(range(len(seqs))), 0, []
    while live:
        sizes.append(len(live))
        got = e.step([StepEntry(slots[i], [seqs[i][prompt_lens[i] + step]], [0]) for i in live]).cpu().numpy()
        for row, i in enumerate(live):
            assert rel_err(got[row], refs[i][1 + step]) < TOL[dtype], f"request {i} position {prompt_lens[i] + step} ({len(live)} rows)"
        step += 1
        for i in list(live):
            if prompt_lens[i] + step >= len(seqs[i]):
                e.close(slots[i])
                live.remove(i)
    assert sorted(set(sizes)) == [1, 2, 3, 4, 5]
    e.cache.book.check_all_free()
    if dtype == "bfloat16" and name == "xl":
        assert e.ops._sums is not None, "the q/k/v product of 3..16 rows was expected to leave 32-bit sums at this K"
