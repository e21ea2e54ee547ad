"""The engine at the layer sizes the benchmark runs - GPT-2 small: width 768, 12 heads of 64, inner
width 3072, vocabulary 50257, 1024 positions - with 2 of GPT-2 small's 12 layers, against the plain
implementation, in 32-bit and in bfloat16, under every cut: whole requests, the last 32 tokens one by
one, unequal batches one after another with slots and pages used again, a batch of 64 sequences that
shrinks through the row counts at which the kernels change form, and a 2 x 1024-token prompt step run
eagerly, captured and replayed.

The model folder is written by tests/plain/fixture.py (real checkpoint layout, stored in 32-bit with
full mantissas), not by the library.  The cache is NaN-poisoned first."""
import numpy as np
import pytest

from kvad_b200 import Engine, StepEntry
from tests.conftest import TOL, random_tokens, rel_err
from tests.plain.fixture import write_gpt2_folder
from tests.plain.gpt2_plain import PlainGpt2

pytestmark = pytest.mark.gpu

SMALL = dict(model_type="gpt2", n_layer=2, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257, n_positions=1024,
             layer_norm_epsilon=1e-5, activation_function="gelu_new")        # GPT-2 small has 12 layers; 2 run here
V, P = SMALL["vocab_size"], SMALL["n_positions"]
CACHE_TOKENS = 21 * 1024          # less than the batches below need together: slots and pages come back and are used again


@pytest.fixture(scope="module")
def small_dir(tmp_path_factory):
    return write_gpt2_folder(str(tmp_path_factory.mktemp("gpt2small2")), SMALL, seed=51, dtype="F32")


@pytest.fixture(scope="module")
def small(small_dir):
    made = {}

    def get(dtype):
        if dtype not in made:
            e = Engine.from_pretrained(small_dir, dtype, max_tokens=CACHE_TOKENS)
            for k, v in e.cache.kv.values():
                k.fill_(float("nan"))
                v.fill_(float("nan"))
            made[dtype] = (e, PlainGpt2(small_dir, round_to="bfloat16" if dtype == "bfloat16" else None))
        return made[dtype]

    return get


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_each_request_alone_and_whole(small, dtype):
    e, plain = small(dtype)
    for i, n in enumerate([1, 64, 65, 513, 1024]):
        t = random_tokens(1000 + i, n, V)
        want = sorted({0, n // 3, max(0, n - 2), n - 1})
        s = e.open()
        got = e.step([StepEntry(s, t, want)]).cpu().numpy()
        e.close(s)
        assert rel_err(got, plain.logits(t, rows=want)) < TOL[dtype], (dtype, n)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_last_32_tokens_one_by_one(small, dtype):
    e, plain = small(dtype)
    t = random_tokens(1010, P, V)
    head = P - 32
    ref = plain.logits(t, rows=[0, 500, head - 1, *range(head, P)])
    s = e.open()
    got = e.step([StepEntry(s, t[:head], [0, 500, head - 1])]).cpu().numpy()
    assert rel_err(got, ref[:3]) < TOL[dtype]
    for j in range(head, P):
        got = e.step([StepEntry(s, [t[j]], [0])]).cpu().numpy()
        assert rel_err(got[0], ref[3 + j - head]) < TOL[dtype], f"{dtype}: first wrong decoded position {j}"
    with pytest.raises(Exception, match="context window"):
        e.step([StepEntry(s, [1], [0])])
    e.close(s)
    e.cache.book.check_all_free()


def _run_batch(e, plain, dtype, seqs, prompt_lens, tag):
    """Prompts in one step, then one token each until every sequence has run out; shorter ones end earlier."""
    refs = [plain.logits(t, rows=range(p - 1, len(t))) for t, p in zip(seqs, prompt_lens)]
    slots = [e.open() for _ in seqs]
    got = e.step([StepEntry(s, t[:p], [p - 1]) for s, t, p in zip(slots, seqs, prompt_lens)]).cpu().numpy()
    for i in range(len(seqs)):
        assert rel_err(got[i], refs[i][0]) < TOL[dtype], f"{tag}: end of prompt {i} ({prompt_lens[i]} tokens)"
    live, step, sizes = list(range(len(seqs))), 0, []
    while True:
        for i in list(live):
            if prompt_lens[i] + step >= len(seqs[i]):
                e.close(slots[i])
                live.remove(i)
        if not live:
            break
        sizes.append(len(live))
        got = e.step([StepEntry(slots[i], [seqs[i][prompt_lens[i] + step]], [0]) for i in live]).cpu().numpy()
        for row, i in enumerate(live):
            assert rel_err(got[row], refs[i][1 + step]) < TOL[dtype], \
                f"{tag}: request {i} position {prompt_lens[i] + step} (decode step {step}, {len(live)} rows)"
        step += 1
    return sizes


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_one_after_another(small, dtype):
    e, plain = small(dtype)
    rng = np.random.default_rng(5)
    # 64 sequences; eight leave after each of the decode steps 8..15: 64, 56, 48, 40, 32, 24, 16 and 8 rows
    prompt_lens = [int(x) for x in rng.integers(20, 300, 64)]
    prompt_lens[:4] = [1, 63, 64, 65]
    seqs = [random_tokens(1100 + i, p + 8 + i // 8, V) for i, p in enumerate(prompt_lens)]
    sizes = _run_batch(e, plain, dtype, seqs, prompt_lens, "batch of 64")
    assert sizes[:8] == [64] * 8 and sorted(set(sizes)) == [8, 16, 24, 32, 40, 48, 56, 64]
    e.cache.book.check_all_free()
    # two prompts of 1024 tokens in one step, three times: launched kernel by kernel, captured, replayed
    for rep in range(3):
        a, b = random_tokens(1200 + rep, P, V), random_tokens(1210 + rep, P, V)
        sa, sb = e.open(), e.open()
        got = e.step([StepEntry(sa, a, [0, 700, P - 1]), StepEntry(sb, b, [P - 1])]).cpu().numpy()
        e.close(sa), e.close(sb)
        assert rel_err(got[:3], plain.logits(a, rows=[0, 700, P - 1])) < TOL[dtype], (dtype, rep)
        assert rel_err(got[3], plain.logits(b, rows=[P - 1])[0]) < TOL[dtype], (dtype, rep)
    if e.use_graphs:
        assert any(k[0] == "step" and k[1] == 2 * P and v != "seen" for k, v in e._graphs.items())
    # a small batch through slots and pages that the batches before gave back
    prompt_lens = [1, 63, 64, 65, 400]
    seqs = [random_tokens(1300 + i, p + x, V) for i, (p, x) in enumerate(zip(prompt_lens, [12, 3, 9, 1, 6]))]
    _run_batch(e, plain, dtype, seqs, prompt_lens, "batch of 5")
    e.cache.book.check_all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_decoding_on_the_device_follows_the_oracle(small, dtype):
    """`decode_run` at 8 sequences from 512-token prompts (the benchmark's own road): every chosen token is,
    within the dtype's tolerance, the oracle's best continuation of the engine's own prefix."""
    e, plain = small(dtype)
    prompts = [random_tokens(1400 + i, 512, V) for i in range(8)]
    slots = [e.open() for _ in prompts]
    first = e.step([StepEntry(s, p, [511]) for s, p in zip(slots, prompts)]).argmax(-1).tolist()
    hist = e.decode_run(slots, first, 6).cpu().numpy()
    for s in slots:
        e.close(s)
    for i in (0, 3, 7):
        out = [first[i]] + hist[:, i].tolist()
        ref = plain.logits(prompts[i] + out, rows=range(511, 511 + len(out)))
        for j, tok in enumerate(out):
            assert ref[j].max() - ref[j][tok] <= 2 * TOL[dtype] * np.abs(ref[j]).max(), (dtype, i, j)
            if dtype == "float32":
                assert tok == int(np.argmax(ref[j])), (i, j)
    e.cache.book.check_all_free()
