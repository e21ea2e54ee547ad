"""The engine against the plain implementation, in 32-bit and in bfloat16, under every way of
cutting the work: whole requests, the last 32 tokens one by one, unequal batches with slot reuse,
long decoding, the first tokens, and greedy generation through the entry point."""
import numpy as np
import pytest
import torch

from kvad_b200 import StepEntry
from tests.conftest import TINY, TOL, random_tokens, rel_err

pytestmark = pytest.mark.gpu
CASES = [(c, d) for c in ("A", "B", "C", "D") for d in ("float32", "bfloat16")]
# folders in real checkpoint layout that the library did not write, stored in 32-bit / float16, sharded
CASES += [("A32", "float32"), ("B32", "float32"), ("B32", "bfloat16"), ("U16", "float32"), ("U16", "bfloat16")]


def poison(engine):
    """Fills the whole cache with NaN: a read outside a sequence's own positions shows at once."""
    for k, v in engine.cache.kv.values():
        k.fill_(float("nan"))
        v.fill_(float("nan"))


def lengths_for(cfg):
    p = cfg["n_positions"]
    return [1, 5, 17, 64, 65, min(p, 127), p]


@pytest.mark.parametrize("name,dtype", CASES)
def test_each_request_alone_and_whole(engines, plains, name, dtype):
    e, plain, cfg = engines(name, dtype), plains(name, dtype), TINY[name]
    poison(e)
    for i, n in enumerate(lengths_for(cfg)):
        t = random_tokens(100 + i, n, cfg["vocab_size"])
        slot = e.open()
        got = e.step([StepEntry(slot, t, range(n))]).cpu().numpy()
        e.close(slot)
        assert rel_err(got, plain.logits(t)) < TOL[dtype], (name, dtype, n)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("name,dtype", CASES)
def test_last_32_tokens_one_by_one(engines, plains, name, dtype):
    e, plain, cfg = engines(name, dtype), plains(name, dtype), TINY[name]
    poison(e)
    for i, n in enumerate([33, 70, cfg["n_positions"]]):
        t = random_tokens(200 + i, n, cfg["vocab_size"])
        ref = plain.logits(t)
        slot = e.open()
        head = n - 32
        got = [e.step([StepEntry(slot, t[:head], range(head))]).cpu().numpy()]
        for j in range(head, n):
            got.append(e.step([StepEntry(slot, [t[j]], [0])]).cpu().numpy())
        e.close(slot)
        got = np.concatenate(got)
        assert rel_err(got[:head], ref[:head]) < TOL[dtype]
        for j in range(head, n):      # find the first wrong token, not just "something is wrong"
            assert rel_err(got[j], ref[j]) < TOL[dtype], f"{name} {dtype}: first wrong decoded position {j} of {n}"
    e.cache.book.check_all_free()


@pytest.mark.parametrize("name,dtype", CASES)
def test_unequal_batches_one_after_another(engines, plains, name, dtype):
    """Prompts of unequal lengths in one step, then one token each; shorter requests end earlier;
    batch after batch through a cache so small that slots and pages are used again."""
    cfg = TINY[name]
    e, plain = engines(name, dtype, max_tokens=512), plains(name, dtype)
    poison(e)
    V, P = cfg["vocab_size"], cfg["n_positions"]
    rng = np.random.default_rng(7)
    for b in range(4):
        prompt_lens = [1, 7, 30, 64][: 3 + b % 2] if b % 2 else [5, 11, 17]
        extra = [int(rng.integers(1, 13)) for _ in prompt_lens]                 # decoded tokens, unequal
        seqs = [random_tokens(300 + 10 * b + i, min(P, p + x), V) for i, (p, x) in enumerate(zip(prompt_lens, extra))]
        refs = [plain.logits(t) for t in seqs]
        slots = [e.open() for _ in seqs]
        got = e.step([StepEntry(s, t[:p], [p - 1]) for s, t, p in zip(slots, seqs, prompt_lens)]).cpu().numpy()
        for i, p in enumerate(prompt_lens):
            assert rel_err(got[i], refs[i][p - 1]) < TOL[dtype], f"batch {b}: end of prompt {i}"
        live = list(range(len(seqs)))
        step = 0
        while True:
            for i in list(live):
                if prompt_lens[i] + step >= len(seqs[i]):
                    e.close(slots[i])                                            # ends earlier; its slot goes back
                    live.remove(i)
            if not live:
                break
            got = e.step([StepEntry(slots[i], [seqs[i][prompt_lens[i] + step]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                pos = prompt_lens[i] + step
                assert rel_err(got[row], refs[i][pos]) < TOL[dtype], f"batch {b}: request {i} position {pos} (decode step {step})"
            step += 1
        e.cache.book.check_all_free()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("B", "float32"), ("B", "bfloat16")])
def test_long_decoding(engines, plains, name, dtype):
    """From a short prompt to the end of the context, one token at a time, two sequences of unequal age."""
    e, plain, cfg = engines(name, dtype), plains(name, dtype), TINY[name]
    poison(e)
    P, V = cfg["n_positions"], cfg["vocab_size"]
    a, b = random_tokens(401, P, V), random_tokens(402, P - 40, V)
    ra, rb = plain.logits(a), plain.logits(b)
    sa, sb = e.open(), e.open()
    got = e.step([StepEntry(sa, a[:3], [2]), StepEntry(sb, b[:1], [0])]).cpu().numpy()
    assert rel_err(got[0], ra[2]) < TOL[dtype] and rel_err(got[1], rb[0]) < TOL[dtype]
    for j in range(P - 3):
        ents = [StepEntry(sa, [a[3 + j]], [0])]
        if 1 + j < len(b):
            ents.append(StepEntry(sb, [b[1 + j]], [0]))
        elif 1 + j == len(b):
            e.close(sb)
        got = e.step(ents).cpu().numpy()
        assert rel_err(got[0], ra[3 + j]) < TOL[dtype], f"sequence a, position {3 + j}"
        if len(ents) == 2:
            assert rel_err(got[1], rb[1 + j]) < TOL[dtype], f"sequence b, position {1 + j}"
    with pytest.raises(Exception, match="context window"):
        e.step([StepEntry(sa, [1], [0])])
    assert e.length(sa) == P                                # the refused step changed nothing
    e.close(sa)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_prompts_in_two_portions_then_decoding_across_page_edges(engines, plains, dtype):
    """Heads of 64, 1024 positions: two prompts given in two portions each (the second continues cached
    positions and crosses a 128-row tile and a page edge), then single tokens across positions 512 and 704."""
    e, plain, cfg = engines("D", dtype, max_tokens=2048), plains("D", dtype), TINY["D"]
    poison(e)
    V = cfg["vocab_size"]
    a, b = random_tokens(450, 716, V), random_tokens(451, 531, V)
    ra, rb = plain.logits(a), plain.logits(b)
    sa, sb = e.open(), e.open()
    got = e.step([StepEntry(sa, a[:333], range(333)), StepEntry(sb, b[:300], range(300))]).cpu().numpy()
    assert rel_err(got[:333], ra[:333]) < TOL[dtype] and rel_err(got[333:], rb[:300]) < TOL[dtype]
    got = e.step([StepEntry(sa, a[333:700], range(367)), StepEntry(sb, b[300:505], range(205))]).cpu().numpy()
    assert rel_err(got[:367], ra[333:700]) < TOL[dtype], "second portion of a"
    assert rel_err(got[367:], rb[300:505]) < TOL[dtype], "second portion of b"
    for j in range(16):
        got = e.step([StepEntry(sa, [a[700 + j]], [0]), StepEntry(sb, [b[505 + j]], [0])]).cpu().numpy()
        assert rel_err(got[0], ra[700 + j]) < TOL[dtype], f"a at {700 + j}"
        assert rel_err(got[1], rb[505 + j]) < TOL[dtype], f"b at {505 + j}"
    e.close(sa)
    for j in range(16, 26):                                  # b alone, past the page edge at 512
        got = e.step([StepEntry(sb, [b[505 + j]], [0])]).cpu().numpy()
        assert rel_err(got[0], rb[505 + j]) < TOL[dtype], f"b at {505 + j}"
    e.close(sb)
    e.cache.book.check_all_free()


@pytest.mark.parametrize("name,dtype", CASES)
def test_first_tokens_of_a_sequence(engines, plains, name, dtype):
    e, plain, cfg = engines(name, dtype), plains(name, dtype), TINY[name]
    t = random_tokens(500, 4, cfg["vocab_size"])
    ref = plain.logits(t)
    slot = e.open()
    for j in range(4):
        got = e.step([StepEntry(slot, [t[j]], [0])]).cpu().numpy()
        assert rel_err(got[0], ref[j]) < TOL[dtype], f"position {j}"
    e.close(slot)
    slot = e.open()                                          # wanting nothing is allowed, and wanting the middle
    assert e.step([StepEntry(slot, t[:2], [])]).shape[0] == 0
    got = e.step([StepEntry(slot, t[2:], [0])]).cpu().numpy()
    assert rel_err(got[0], ref[2]) < TOL[dtype]
    e.close(slot)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_cutting_changes_nothing_in_32_bit(engines, name):
    """The same positions through different cuts and different company: equal to rounding, far below the
    distance to the oracle."""
    e, cfg = engines(name, "float32"), TINY[name]
    V = cfg["vocab_size"]
    t, u = random_tokens(600, 90, V), random_tokens(601, 41, V)
    s = e.open()
    whole = e.step([StepEntry(s, t, range(90))]).cpu().numpy()
    e.close(s)
    s, s2 = e.open(), e.open()
    parts = [e.step([StepEntry(s, t[:50], range(50)), StepEntry(s2, u, [40])]).cpu().numpy()[:50],
             e.step([StepEntry(s, t[50:77], range(27))]).cpu().numpy()]
    for j in range(77, 90):
        parts.append(e.step([StepEntry(s2, [u[j % 41]], []), StepEntry(s, [t[j]], [0])]).cpu().numpy())
    e.close(s), e.close(s2)
    assert rel_err(np.concatenate(parts), whole) < 2e-6


@pytest.mark.parametrize("name,dtype", CASES)
def test_greedy_generation_through_the_entry_point(engines, plains, model_dirs, name, dtype):
    """Engine.generate, greedy, against the oracle: every token the engine chose is (within the dtype's
    tolerance) the oracle's best continuation of the engine's own prefix."""
    from tests.plain.gpt2_plain import PlainGpt2
    e, cfg = engines(name, dtype), TINY[name]
    from tests.conftest import FOREIGN
    # the float64 oracle on the stored values; where a bfloat16 engine holds other values than the file
    # stores (a 32-bit or float16 file), the oracle that rounds as the engine does
    oracle = plains(name, dtype) if (name in FOREIGN and dtype == "bfloat16") else PlainGpt2(model_dirs[name])
    prompts = [random_tokens(700 + i, n, cfg["vocab_size"]) for i, n in enumerate([5, 11, 17])]
    outs = e.generate(prompts, max_tokens=8, temperature=0.0)
    e.cache.book.check_all_free()
    exact = 0
    for p, o in zip(prompts, outs):
        assert len(o) == 8
        ref = oracle.logits(p + o)
        for j, tok in enumerate(o):
            row = ref[len(p) - 1 + j]
            exact += int(tok == int(np.argmax(row)))
            assert row.max() - row[tok] <= TOL[dtype] * np.abs(row).max() * 2, f"token {j} of prompt {len(p)}"
    if dtype == "float32":
        assert exact == 24
    # batches one after another give the same tokens as all at once.  In 32-bit that is exact (a row's bits do not
    # depend on its company); in bfloat16 the residual products add their K splits with atomics, so logits can
    # differ in the last bit between runs and a near tie may fall the other way: there the tokens must still be
    # the oracle's best within the tolerance.
    again = e.generate(prompts, max_tokens=8, temperature=0.0, batch_size=2)
    if dtype == "float32":
        assert again == outs
    else:
        for p, o in zip(prompts, again):
            ref = oracle.logits(p + o)
            for j, tok in enumerate(o):
                row = ref[len(p) - 1 + j]
                assert row.max() - row[tok] <= TOL[dtype] * np.abs(row).max() * 2, f"second run: token {j} of prompt {len(p)}"


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("B", "bfloat16"), ("D", "bfloat16")])
def test_decode_run_gives_the_tokens_of_generate(engines, plains, model_dirs, name, dtype):
    """`Engine.decode_run` (decoding with the chosen tokens fed back on the device, the road the benchmark
    times) chooses the same tokens as `Engine.generate`, and in 32-bit they are the oracle's greedy tokens."""
    e, cfg = engines(name, dtype), TINY[name]
    prompts = [random_tokens(720 + i, n, cfg["vocab_size"]) for i, n in enumerate([9, 4, 15, 6, 1])]
    want = e.generate(prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    slots = [e.open() for _ in prompts]
    logits = e.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, prompts)])
    first = logits.argmax(-1).tolist()
    hist = e.decode_run(slots, first, 11).cpu().numpy()
    for s in slots:
        e.close(s)
    e.cache.book.check_all_free()
    got = [[first[i]] + hist[:, i].tolist() for i in range(len(prompts))]
    assert got == want
    if dtype == "float32":
        oracle = plains(name, dtype)
        for p, o in zip(prompts, got):
            assert o == oracle.greedy(p, 12), len(p)


def test_stop_token_and_unequal_ends(engines, plains):
    e = engines("A", "float32")
    p = [random_tokens(800, 6, 512), random_tokens(801, 9, 512)]
    free = e.generate(p, max_tokens=10, temperature=0.0)
    stop = free[0][3]
    outs = e.generate(p, max_tokens=10, temperature=0.0, stop_token_ids=[stop])
    cut0 = free[0].index(stop)
    assert outs[0] == free[0][:cut0] and stop not in outs[0]
    assert outs[1] == (free[1][:free[1].index(stop)] if stop in free[1] else free[1])
    e.cache.book.check_all_free()


def test_refusals_change_nothing(engines):
    e = engines("A", "float32", max_tokens=128)
    s = e.open()
    e.step([StepEntry(s, [1, 2, 3], [])])
    for bad in ([StepEntry(s, [512], [0])], [StepEntry(s, [], [])], [StepEntry(s, [1], [1])], [StepEntry(99, [1], [0])]):
        with pytest.raises(Exception):
            e.step(bad)
    s2 = e.open()
    with pytest.raises(Exception, match="cache is full"):
        e.step([StepEntry(s, [1] * 60, []), StepEntry(s2, [2] * 70, [])])      # 2 pages for s2, only 1 left
    assert e.length(s) == 3 and e.length(s2) == 0
    e.close(s), e.close(s2)
    e.cache.book.check_all_free()


def test_no_cpu_path(model_dirs):
    from kvad_b200.ops import KernelError, Ops
    ops = Ops(torch.float32)
    x = torch.zeros(2, 8)
    with pytest.raises(KernelError, match="no CPU path"):
        ops.layernorm(x, torch.ones(8), None, 1e-5, torch.zeros(2, 8))


@pytest.mark.parametrize("n_layer", [2, 3])
def test_qkv_as_32_bit_sums_finished_by_the_attention_kernel(tmp_path, n_layer):
    """The decode form that long K takes (the q/k/v product adds into a 32-bit buffer, the attention kernel adds
    the bias, rounds and writes the cache), forced at a tiny size: 3 to 5 rows, unequal lengths, sequences that
    end earlier, an odd number of layers (the first buffer is cleared at the step's end) and an even one, every
    step shape kernel by kernel the first time and as a replayed graph afterwards."""
    from kvad_b200 import Engine, write_random_model
    from tests.plain.gpt2_plain import PlainGpt2
    cfg = dict(model_type="gpt2", n_layer=n_layer, n_embd=128, n_head=2, n_inner=320, vocab_size=700, n_positions=512,
               layer_norm_epsilon=1e-5, activation_function="gelu_new")
    write_random_model(str(tmp_path), cfg, seed=77 + n_layer)
    e, plain = Engine.from_pretrained(str(tmp_path), "bfloat16", max_tokens=2048), PlainGpt2(str(tmp_path), round_to="bfloat16")
    e.ops.SUMS_MIN_K = 0
    poison(e)
    V = cfg["vocab_size"]
    for b, prompt_lens in enumerate(([5, 11, 17], [1, 7, 30, 64, 3], [9, 2, 33, 4])):
        seqs = [random_tokens(700 + 10 * b + i, p + 6 + 2 * i, V) for i, p in enumerate(prompt_lens)]
        refs = [plain.logits(t) for t in seqs]
        slots = [e.open() for _ in seqs]
        e.step([StepEntry(s, t[:p], []) for s, t, p in zip(slots, seqs, prompt_lens)])
        live, step = list(range(len(seqs))), 0
        while live:
            got = e.step([StepEntry(slots[i], [seqs[i][prompt_lens[i] + step]], [0]) for i in live]).cpu().numpy()
            for row, i in enumerate(live):
                pos = prompt_lens[i] + step
                assert rel_err(got[row], refs[i][pos]) < TOL["bfloat16"], f"batch {b}: request {i} position {pos} ({len(live)} rows)"
            step += 1
            for i in list(live):
                if prompt_lens[i] + step >= len(seqs[i]):
                    e.close(slots[i])
                    live.remove(i)
        e.cache.book.check_all_free()
    assert e.ops._sums is not None, "the form under test did not run"
    assert float(e.ops._sums[0].abs().sum()) == 0.0      # clean for the next step: by the last reader, or by the step's end


def test_dependent_launch_changes_no_result(engines, plains):
    """Kernels may start before the one before them has finished (they wait before touching its output):
    the 32-bit logits are the same bits with that switched off, and the bfloat16 ones stay right."""
    from kvad_b200 import ops
    t = random_tokens(950, 100, 512)
    outs = {}
    try:
        for on in (True, False):
            ops.set_pdl(on)                         # a new switch epoch: no graph captured under the other setting is replayed
            for dtype in ("float32", "bfloat16"):
                e = engines("A", dtype)
                assert not any(k[-1] == e.ops.path_key() for k in e._graphs), "a graph of the other arm would be replayed"
                s = e.open()
                got = [e.step([StepEntry(s, t[:90], range(90))]).cpu().numpy()]
                for j in range(90, 100):
                    got.append(e.step([StepEntry(s, [t[j]], [0])]).cpu().numpy())
                e.close(s)
                outs[(on, dtype)] = np.concatenate(got)
    finally:
        ops.set_pdl(True)
    assert np.array_equal(outs[(True, "float32")], outs[(False, "float32")])
    ref = plains("A", "bfloat16").logits(t)
    assert rel_err(outs[(True, "bfloat16")], ref) < TOL["bfloat16"] and rel_err(outs[(False, "bfloat16")], ref) < TOL["bfloat16"]


def test_repeated_step_shapes_replay_a_graph_with_the_same_result(engines, plains):
    """The second prompt step of a shape is captured, the third replays: all three give the oracle's logits,
    although positions, lengths and pages differ between them."""
    e, plain = engines("B", "bfloat16"), plains("B", "bfloat16")
    assert e.use_graphs
    before = len([v for v in e._graphs.values() if v != "seen"])
    for rep in range(4):
        a, b = random_tokens(970 + rep, 50, 1000), random_tokens(980 + rep, 21, 1000)
        sa, sb = e.open(), e.open()
        pre = 7 * rep                                  # the same shape of step at other positions
        if pre:
            e.step([StepEntry(sa, a[:pre], []), StepEntry(sb, b[:1], [])])
        got = e.step([StepEntry(sa, a[pre:pre + 20], [19]), StepEntry(sb, b[1 if pre else 0:][:20], [0, 19])]).cpu().numpy()
        off = 1 if pre else 0
        ref = np.stack([plain.logits(a[:pre + 20])[pre + 19], plain.logits(b[:off + 20])[off], plain.logits(b[:off + 20])[off + 19]])
        assert rel_err(got, ref) < TOL["bfloat16"], rep
        e.close(sa), e.close(sb)
    assert len([v for v in e._graphs.values() if v != "seen"]) > before


def test_random_weights_entry_point(tmp_path):
    """Engine.random writes a model folder from a configuration and a seed and loads it like any other: the folder
    it leaves gives the plain implementation the same weights, and the same seed gives the same model without one."""
    from kvad_b200 import Engine
    from tests.plain.gpt2_plain import PlainGpt2
    d = str(tmp_path / "m")
    e = Engine.random(TINY["B"], seed=5, dtype="float32", model_dir=d, max_tokens=1024)
    plain = PlainGpt2(d)
    prompt = random_tokens(3, 11, TINY["B"]["vocab_size"])
    got = e.generate([prompt], max_tokens=6, temperature=0.0, stop_token_ids=[])[0]
    seq = list(prompt)
    for _ in range(6):
        seq.append(int(np.argmax(plain.logits(seq)[-1])))
    assert got == seq[len(prompt):]
    again = Engine.random(TINY["B"], seed=5, dtype="float32", max_tokens=1024)
    assert again.generate([prompt], max_tokens=6, temperature=0.0, stop_token_ids=[])[0] == got
    other = Engine.random(TINY["B"], seed=6, dtype="float32", max_tokens=1024)
    assert other.generate([prompt], max_tokens=6, temperature=0.0, stop_token_ids=[])[0] != got


def test_random_weights_stored_in_32_bit(tmp_path):
    """The random-weights mode storing float32: the 32-bit engine multiplies by values bfloat16 cannot hold."""
    from kvad_b200 import Engine, write_random_model
    from tests.plain.gpt2_plain import PlainGpt2, round_bf16
    d = str(tmp_path / "m32")
    write_random_model(d, TINY["B"], 9, store_dtype="float32")
    plain = PlainGpt2(d)
    w = plain.w["h.0.mlp.c_fc.weight"]
    assert np.mean(round_bf16(w) != w) > 0.9
    e = Engine.from_pretrained(d, "float32", max_tokens=512)
    t = random_tokens(12, 80, TINY["B"]["vocab_size"])
    ref = plain.logits(t)
    s = e.open()
    got = [e.step([StepEntry(s, t[:70], range(70))]).cpu().numpy()]
    for j in range(70, 80):
        got.append(e.step([StepEntry(s, [t[j]], [0])]).cpu().numpy())
    e.close(s)
    assert rel_err(np.concatenate(got), ref) < TOL["float32"]
