"""Each kernel alone against a plain reference of the same operation (float64 on the CPU, from the
same inputs), at sizes other than the engine's: widths and vocabularies that are no power of two,
head sizes in steps of 16, grouped heads, windows, strided inputs, and inputs made so that a fault
cannot hide (one far key whose score stands out, a window's edge)."""
import math

import numpy as np
import pytest
import torch

from kvad_b200.ops import KernelError, Ops

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# element-wise closeness of a kernel's output to the float64 reference, relative to the largest value
KTOL = {"float32": 3e-6, "bfloat16": 6e-3}


def dev(t):
    return t.to("cuda")


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert torch.isfinite(got).all()
    return float((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30))


def gelu_tanh(v):
    return 0.5 * v * (1 + torch.tanh(math.sqrt(2 / math.pi) * (v + 0.044715 * v ** 3)))


def gelu_erf(v):
    return 0.5 * v * (1 + torch.erf(v / math.sqrt(2)))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width,vocab,npos", [(48, 1031, 77), (1600, 257, 1024), (8, 5, 3)])
def test_embed(dtype, width, vocab, npos):
    g = torch.Generator().manual_seed(1)
    ops = Ops(DT[dtype])
    wte, wpe = torch.randn(vocab, width, generator=g).to(DT[dtype]), torch.randn(npos, width, generator=g).to(DT[dtype])
    n = 37
    tok = torch.randint(0, vocab, (n,), generator=g, dtype=torch.int32)
    pos = torch.randint(0, npos, (n,), generator=g, dtype=torch.int32)
    tok[0], tok[1], pos[0], pos[1] = 0, vocab - 1, npos - 1, 0
    out = torch.full((n, width), float("nan"), device="cuda")
    ops.embed(dev(tok), dev(pos), dev(wte), dev(wpe), out)
    assert torch.equal(out.cpu(), wte.float()[tok.long()] + wpe.float()[pos.long()])      # one 32-bit add: exact
    ops.embed(dev(tok), dev(pos), dev(wte), None, out)
    assert torch.equal(out.cpu(), wte.float()[tok.long()])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [16, 80, 1024, 1032, 1600, 4096, 4104, 5000])      # a warp per row / four warps per row / a block per row through shared memory
def test_layernorm(dtype, width):
    g = torch.Generator().manual_seed(2)
    ops = Ops(DT[dtype])
    n = 9
    x = torch.randn(n, width, generator=g) * 3 + 1.5
    gain, bias = torch.randn(width, generator=g), torch.randn(width, generator=g)
    eps = 1e-3

    def ref(rows, gn, bs):
        xr = x.double()[rows]
        mean = xr.mean(-1, keepdim=True)
        var = ((xr - mean) ** 2).mean(-1, keepdim=True)
        return (xr - mean) / torch.sqrt(var + eps) * gn.double() + (bs.double() if bs is not None else 0)

    for params in ("same", "f32"):                       # parameters in the compute dtype, or kept in 32-bit
        gn = gain.to(DT[dtype]) if params == "same" else gain
        bs = bias.to(DT[dtype]) if params == "same" else bias
        out = torch.full((n, width), float("nan"), device="cuda", dtype=DT[dtype])
        ops.layernorm(dev(x), dev(gn), dev(bs), eps, out)
        assert rel(out, ref(torch.arange(n), gn, bs)) < KTOL[dtype]
    rows = torch.tensor([7, 0, 7, 3], dtype=torch.int32)
    out = torch.full((4, width), float("nan"), device="cuda", dtype=DT[dtype])
    ops.layernorm(dev(x), dev(gain.to(DT[dtype])), None, eps, out, dev(rows))
    assert rel(out, ref(rows.long(), gain.to(DT[dtype]), None)) < KTOL[dtype]


def linear_case(ops, dtype, m, n, k, epilogue, g, *, bias=True, strided=False, bias_f32=False, **kw):
    a = torch.randn(m, k + (8 if strided else 0), generator=g).to(DT[dtype])
    w = (torch.randn(n, k, generator=g) / math.sqrt(k)).to(DT[dtype])
    b = torch.randn(n, generator=g) if bias else None
    if b is not None and not bias_f32:
        b = b.to(DT[dtype])
    a_dev = dev(a)[:, :k] if strided else dev(a)
    ref = a[:, :k].double() @ w.double().t() + (b.double() if b is not None else 0)
    if epilogue == "gelu_tanh":
        ref = gelu_tanh(ref)
    elif epilogue == "gelu_erf":
        ref = gelu_erf(ref)
    if epilogue == "residual":
        base = torch.randn(m, n, generator=g)
        out = dev(base.clone())
        ref = ref + base.double()
    elif epilogue == "store_f32":
        out = torch.full((m, n), float("nan"), device="cuda")
    else:
        out = torch.full((m, n), float("nan"), device="cuda", dtype=DT[dtype])
    ops.linear(a_dev, dev(w), None if b is None else dev(b), out, epilogue, **kw)
    return rel(out, ref)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_linear_cuda_cores(dtype):
    ops = Ops(DT[dtype])
    ops.tensor_core_linear = False
    ops.rows_linear_max = 0                 # every row count on the tiled kernel
    g = torch.Generator().manual_seed(3)
    # odd shapes of bisand/kvad's own GEMM test (crates/llm/src/tensor.rs:487-500) and larger ones
    for m, n, k in [(9, 13, 7), (8, 16, 4), (5, 32, 1), (6, 8, 9), (1, 1031, 200), (130, 70, 333), (64, 64, 16)]:
        for epi in ("store", "gelu_tanh", "gelu_erf", "residual", "store_f32"):
            assert linear_case(ops, dtype, m, n, k, epi, g) < KTOL[dtype], (m, n, k, epi)
    assert linear_case(ops, dtype, 7, 19, 24, "store", g, bias=False, strided=True) < KTOL[dtype]
    assert linear_case(ops, dtype, 7, 19, 24, "store_f32", g, bias_f32=True) < KTOL[dtype]


def test_linear_is_true_32_bit_and_row_independent():
    """The 32-bit kernels sum with fused multiply-adds in an order that depends on K only: a row gives the same
    bits whatever its company, on each of the two roads (at most 16 rows: the weight stream; more: the tiled
    kernel, 64 x 64 or 128 x 128 tiles); the two roads agree to rounding; and values that a 19-bit (TF32)
    product would lose survive on both."""
    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(4)
    a, w = torch.randn(300, 96, generator=g), torch.randn(6000, 96, generator=g)

    def run(rows):
        out = torch.empty(len(rows), 6000, device="cuda")
        ops.linear(dev(a[rows]), dev(w), None, out, "store_f32")
        return out

    big = run(list(range(300)))                           # 128 x 128 tiles
    mid = run(list(range(20, 90)))                        # 64 x 64 tiles
    assert torch.equal(big[33:34], mid[13:14])
    few, one = run(list(range(30, 39))), run([33])        # the weight stream, 9 rows and 1
    assert torch.equal(few[3:4], one)
    # the two roads add in another order: equal to rounding, not to the bit
    assert ((one - big[33:34]).abs().max() / big[33].abs().max()).item() < 2e-6
    for m in (1, 40):
        a1 = torch.full((m, 8), 1.0 + 2.0 ** -20)
        w1 = torch.full((1, 8), 1.0 + 2.0 ** -20)
        out = torch.empty(m, 1, device="cuda")
        ops.linear(dev(a1), dev(w1), None, out, "store_f32")
        assert abs(out[0, 0].item() - 8 * (1 + 2.0 ** -20) ** 2) < 2e-6        # TF32 would give exactly 8


@pytest.mark.parametrize("m", [1, 3, 8, 64, 127, 129, 300])
def test_linear_tensor_cores_shapes(m):
    ops = Ops(torch.bfloat16)
    if not ops.tensor_core_linear:
        pytest.skip("tensor-core linear kernel not built")
    from kvad_b200.ops import tcgen05_wait_timeouts
    g = torch.Generator().manual_seed(5 + m)
    # (the last three: K long enough that the few-rows form splits it in 7 (a cluster), 25 and 32)
    for n, k in [(768, 768), (1000, 96), (50, 320), (2304, 64), (16, 3072), (777, 200), (1031, 1600), (4800, 1600), (1600, 6400), (200, 8192)]:
        for epi in ("store", "gelu_tanh", "gelu_erf", "residual", "store_f32"):
            assert linear_case(ops, "bfloat16", m, n, k, epi, g) < KTOL["bfloat16"], (m, n, k, epi)
    assert linear_case(ops, "bfloat16", m, 333, 128, "store", g, bias=False, strided=True) < KTOL["bfloat16"]
    assert linear_case(ops, "bfloat16", m, 333, 128, "residual", g, bias_f32=True) < KTOL["bfloat16"]
    assert tcgen05_wait_timeouts() == 0


@pytest.mark.parametrize("stores", ["tma", "plain"])
@pytest.mark.parametrize("tile", [16, 32, 64, 128, 192, 256])
def test_linear_tensor_cores_every_tile_and_split(tile, stores):
    """Every tile width of the wide form, every split of K, output by TMA store / reduce-add and by plain stores."""
    ops = Ops(torch.bfloat16)
    if not ops.tensor_core_linear:
        pytest.skip("tensor-core linear kernel not built")
    from kvad_b200.ops import tcgen05_plain_stores
    tcgen05_plain_stores(stores == "plain")
    try:
        _every_tile_and_split(ops, tile)
    finally:
        tcgen05_plain_stores(False)


def _every_tile_and_split(ops, tile):
    from kvad_b200.ops import tcgen05_wait_timeouts
    g = torch.Generator().manual_seed(50 + tile)
    for m, n, k in [(5, 1000, 96), (200, 515, 832), (130, 257, 3072), (300, 768, 128), (129, 1024, 64)]:
        for epi in ("store", "gelu_tanh", "gelu_erf", "residual", "store_f32"):
            assert linear_case(ops, "bfloat16", m, n, k, epi, g, tile=tile, form="wide") < KTOL["bfloat16"], (m, n, k, epi)
        for splits in (1, 2, 3, 7):
            assert linear_case(ops, "bfloat16", m, n, k, "residual", g, tile=tile, splits=splits, form="wide") < KTOL["bfloat16"], (m, n, k, splits)
    assert tcgen05_wait_timeouts() == 0


@pytest.mark.parametrize("m", [1, 2, 8, 16, 17, 32, 33, 64])
def test_linear_tensor_cores_swapped_form(m):
    """Few rows: the weights sit on the M side of the MMA.  Same answers as the wide form, at every split."""
    ops = Ops(torch.bfloat16)
    if not ops.tensor_core_linear:
        pytest.skip("tensor-core linear kernel not built")
    from kvad_b200.ops import tcgen05_cluster_k, tcgen05_load_form, tcgen05_wait_timeouts
    g = torch.Generator().manual_seed(70 + m)
    for n, k in [(768, 768), (1000, 96), (50, 320), (2304, 64), (777, 3072), (50257, 768)]:
        for epi in ("store", "gelu_tanh", "gelu_erf", "residual", "store_f32"):
            try:
                for mode in (0, 1, 2):        # the kernel's choice; one load per K block; grouped 3-D loads
                    tcgen05_load_form(mode)
                    assert linear_case(ops, "bfloat16", m, n, k, epi, g, form="swapped") < KTOL["bfloat16"], (m, n, k, epi, mode)
            finally:
                tcgen05_load_form(0)
            for tile in (64, 128):          # weight rows per CTA
                assert linear_case(ops, "bfloat16", m, n, k, epi, g, form="swapped", tile=tile) < KTOL["bfloat16"], (m, n, k, epi, tile)
        for splits in (1, 2, 5, 16):
            assert linear_case(ops, "bfloat16", m, n, k, "residual", g, form="swapped", splits=splits) < KTOL["bfloat16"]
        # storing epilogues: K over the CTAs of a cluster (1, 2, 4 or 8 of them), and kept whole
        for epi in ("store", "gelu_tanh", "store_f32"):
            for splits in (2, 4, 8):
                assert linear_case(ops, "bfloat16", m, n, k, epi, g, form="swapped", splits=splits) < KTOL["bfloat16"], (m, n, k, epi, splits)
            try:
                tcgen05_cluster_k(False)
                assert linear_case(ops, "bfloat16", m, n, k, epi, g, form="swapped") < KTOL["bfloat16"], (m, n, k, epi)
            finally:
                tcgen05_cluster_k(True)
    assert linear_case(ops, "bfloat16", m, 333, 128, "store", g, bias=False, strided=True, form="swapped") < KTOL["bfloat16"]
    assert linear_case(ops, "bfloat16", m, 333, 128, "store_f32", g, bias_f32=True, form="swapped") < KTOL["bfloat16"]
    assert linear_case(ops, "bfloat16", m, 333, 128, "store", g, form="wide") < KTOL["bfloat16"]
    assert tcgen05_wait_timeouts() == 0


def test_linear_tensor_cores_large_and_fallback():
    ops = Ops(torch.bfloat16)
    if not ops.tensor_core_linear:
        pytest.skip("tensor-core linear kernel not built")
    g = torch.Generator().manual_seed(6)
    assert linear_case(ops, "bfloat16", 2048, 2304, 768, "store", g) < KTOL["bfloat16"]
    assert linear_case(ops, "bfloat16", 2, 50257, 768, "store_f32", g, bias=False) < KTOL["bfloat16"]
    # K that TMA cannot stride (not a multiple of 8) goes to the CUDA-core kernel: same answer
    assert linear_case(ops, "bfloat16", 9, 40, 100, "store", g) < KTOL["bfloat16"]
    assert linear_case(ops, "bfloat16", 9, 40, 7, "gelu_erf", g) < KTOL["bfloat16"]


def make_cache(g, dtype, n_seqs, lens, n_kv, hd, page=64, shuffle=True):
    """Random keys/values per sequence, scattered over shuffled pages; returns both the paged tensors and the dense ones."""
    pages_per = [-(-l // page) for l in lens]
    n_pages = sum(pages_per) + 3
    order = torch.randperm(n_pages, generator=g).tolist() if shuffle else list(range(n_pages))
    width = max(pages_per)
    table = torch.full((n_seqs, width), -1, dtype=torch.int32)
    kp = torch.full((n_pages, n_kv, page, hd), float("nan")).to(DT[dtype])
    vp = torch.full((n_pages, n_kv, page, hd), float("nan")).to(DT[dtype])
    ks, vs = [], []
    it = iter(order)
    for s, l in enumerate(lens):
        k = torch.randn(l, n_kv, hd, generator=g).to(DT[dtype])
        v = torch.randn(l, n_kv, hd, generator=g).to(DT[dtype])
        ks.append(k), vs.append(v)
        for p in range(pages_per[s]):
            pid = next(it)
            table[s, p] = pid
            chunk = slice(p * page, min(l, (p + 1) * page))
            kp[pid, :, : chunk.stop - chunk.start] = k[chunk].transpose(0, 1)
            vp[pid, :, : chunk.stop - chunk.start] = v[chunk].transpose(0, 1)
    return table, kp, vp, ks, vs


def attention_ref(q, ks, vs, row_seq, row_pos, n_heads, scale, window):
    n, hd = q.shape[0], ks[0].shape[-1]
    n_kv = ks[0].shape[1]
    out = torch.zeros(n, n_heads * hd, dtype=torch.float64)
    for r in range(n):
        s, p = int(row_seq[r]), int(row_pos[r])
        lo = max(0, p - window + 1) if window else 0
        for h in range(n_heads):
            kv = h // (n_heads // n_kv)
            k, v = ks[s][lo:p + 1, kv].double(), vs[s][lo:p + 1, kv].double()
            w = torch.softmax((k @ q[r, h * hd:(h + 1) * hd].double()) * scale, 0)
            out[r, h * hd:(h + 1) * hd] = w @ v
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,n_heads,n_kv,window", [(16, 4, 4, 0), (48, 6, 2, 0), (80, 3, 1, 0), (128, 2, 2, 50),
                                                    (256, 2, 1, 0), (32, 5, 5, 64)])
def test_kv_store_and_attention(dtype, hd, n_heads, n_kv, window):
    g = torch.Generator().manual_seed(hd + n_heads)
    ops = Ops(DT[dtype])
    lens = [200, 1, 65, 130]
    table, kp, vp, ks, vs = make_cache(g, dtype, 4, lens, n_kv, hd)
    # rows: the last 3 positions of sequence 0, the only one of sequence 1, all of sequence 2, two of sequence 3
    rows = [(0, p) for p in (197, 198, 199)] + [(1, 0)] + [(2, p) for p in range(65)] + [(3, 63), (3, 129)]
    row_seq = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    row_pos = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    n = len(rows)
    # kv_store: write these rows' keys/values from a strided buffer into cleared pages, expect the same pages back
    qkv = torch.randn(n, (n_heads + 2 * n_kv) * hd + 8, generator=g).to(DT[dtype])
    qw, kw = n_heads * hd, n_kv * hd
    for i, (s, p) in enumerate(rows):
        qkv[i, qw:qw + kw] = ks[s][p].reshape(-1)
        qkv[i, qw + kw:qw + 2 * kw] = vs[s][p].reshape(-1)
    kp2, vp2 = kp.clone(), vp.clone()
    for i, (s, p) in enumerate(rows):
        kp2[table[s, p // 64], :, p % 64] = 0
        vp2[table[s, p // 64], :, p % 64] = 0
    qkv_d, kp_d, vp_d, table_d = dev(qkv), dev(kp2), dev(vp2), dev(table)
    ops.kv_store(qkv_d[:, qw:qw + kw], qkv_d[:, qw + kw:qw + 2 * kw], dev(row_seq), dev(row_pos), table_d, kp_d, vp_d)
    same = lambda a, b: torch.equal(torch.nan_to_num(a.float().cpu(), nan=7.0), torch.nan_to_num(b.float(), nan=7.0))
    assert same(kp_d, kp) and same(vp_d, vp)
    out = torch.full((n, qw), float("nan"), device="cuda", dtype=DT[dtype])
    scale = 0.7 / math.sqrt(hd)
    ops.attention(qkv_d[:, :qw], out, dev(row_seq), dev(row_pos), table_d, kp_d, vp_d, n_heads, scale, window)
    ref = attention_ref(qkv[:, :qw], ks, vs, row_seq, row_pos, n_heads, scale, window)
    assert rel(out, ref) < KTOL[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_one_far_key_and_respects_the_window_edge(dtype):
    """One key among 700 is made to stand out (its score is ~30 above the rest): the output must be its value.
    Then a window that ends one short of it must not see it."""
    g = torch.Generator().manual_seed(9)
    ops = Ops(DT[dtype])
    hd, n = 32, 700
    table, kp, vp, ks, vs = make_cache(g, dtype, 1, [n], 1, hd)
    far = 3
    q = torch.randn(1, hd, generator=g).to(DT[dtype])
    key = (q[0].float() * 30.0 / q[0].float().pow(2).sum()).to(DT[dtype])      # q . key ~ 30
    ks[0][far, 0] = key
    ks[0][:, 0][torch.arange(n) != far] *= 0.05
    vs[0][far, 0] = torch.arange(hd).to(DT[dtype])
    table, kp, vp, _, _ = rebuild(table, kp, vp, ks, vs)
    row_seq, row_pos = torch.zeros(1, dtype=torch.int32), torch.tensor([n - 1], dtype=torch.int32)
    out = torch.empty(1, hd, device="cuda", dtype=DT[dtype])
    args = (dev(q), out, dev(row_seq), dev(row_pos), dev(table), dev(kp), dev(vp), 1, 1.0)
    ops.attention(*args, 0)
    ref = attention_ref(q, ks, vs, row_seq, row_pos, 1, 1.0, 0)
    assert rel(out, ref) < KTOL[dtype]
    assert (out.float().cpu()[0] - torch.arange(hd)).abs().max() < 0.05 * hd         # it is that key's value
    ops.attention(*args, n - far)                                                     # window reaches exactly to `far`
    assert (out.float().cpu()[0] - torch.arange(hd)).abs().max() < 0.05 * hd
    ops.attention(*args, n - far - 1)                                                 # one short: gone
    assert rel(out, attention_ref(q, ks, vs, row_seq, row_pos, 1, 1.0, n - far - 1)) < KTOL[dtype]
    assert (out.float().cpu()[0] - torch.arange(hd)).abs().max() > 5


def rebuild(table, kp, vp, ks, vs, page=64):
    for s, (k, v) in enumerate(zip(ks, vs)):
        for p in range(-(-k.shape[0] // page)):
            chunk = slice(p * page, min(k.shape[0], (p + 1) * page))
            kp[table[s, p], :, : chunk.stop - chunk.start] = k[chunk].transpose(0, 1)
            vp[table[s, p], :, : chunk.stop - chunk.start] = v[chunk].transpose(0, 1)
    return table, kp, vp, ks, vs


def test_attention_refuses_what_it_cannot_do():
    ops = Ops(torch.float32)
    kp = torch.zeros(2, 3, 64, 16, device="cuda")
    q = torch.zeros(1, 4 * 16, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    with pytest.raises(KernelError, match="do not divide"):
        ops.attention(q, q.clone(), z, z, torch.zeros(1, 1, dtype=torch.int32, device="cuda"), kp, kp, 4, 1.0)
    kp = torch.zeros(2, 1, 64, 528, device="cuda")
    q = torch.zeros(1, 528, device="cuda")
    with pytest.raises(KernelError, match="head size 528"):
        ops.attention(q, q.clone(), z, z, torch.zeros(1, 1, dtype=torch.int32, device="cuda"), kp, kp, 1, 1.0)


def test_argmax_first_of_equals_and_nan():
    ops = Ops(torch.float32)
    g = torch.Generator().manual_seed(10)
    logits = torch.randn(6, 50257, generator=g)
    logits[1, 40000] = logits[1, 123] = 9.0
    logits[2, :] = -1.0
    logits[3, 7] = float("nan")
    logits[3, 50000] = 8.0
    logits[4, 50256] = 99.0
    buf = torch.zeros(6, 50264, device="cuda")                    # a padded leading dimension
    buf[:, :50257] = dev(logits)
    out = torch.full((6,), -1, dtype=torch.int32, device="cuda")
    ops.argmax(buf[:, :50257], out)
    want = [int(logits[0].argmax()), 123, 0, 50000, 50256, int(logits[5].argmax())]
    assert out.cpu().tolist() == want
    out.fill_(-1)                                                  # the two-stage form agrees
    ops.argmax(buf[:, :50257], out, torch.zeros(6 * 25, dtype=torch.int64, device="cuda"))
    assert out.cpu().tolist() == want
    small = torch.tensor([[1.0, 5.0, 5.0], [float("nan")] * 3], device="cuda")
    out2 = torch.full((2,), -1, dtype=torch.int32, device="cuda")
    ops.argmax(small, out2, torch.zeros(2, dtype=torch.int64, device="cuda"))
    assert out2.cpu().tolist() == [1, 0]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,n_heads,n_kv,window", [(16, 4, 4, 0), (48, 6, 2, 0), (64, 12, 12, 0), (80, 3, 1, 0),
                                                    (128, 2, 2, 50), (256, 2, 1, 0), (32, 5, 5, 64), (112, 2, 2, 0)])
@pytest.mark.parametrize("form", ["tma", "registers", "tma-no-cluster"])
def test_attention_decode_split_keys(dtype, hd, n_heads, n_kv, window, form):
    """The decode kernel (both of its forms) at every split count gives what the plain reference gives; sequences
    of very unequal length share a launch (an empty split, a single key, a page boundary)."""
    from kvad_b200.ops import decode_force_plain, decode_wait_timeouts
    g = torch.Generator().manual_seed(7 * hd + n_heads)
    ops = Ops(DT[dtype])
    decode_force_plain({"tma": 0, "registers": 1, "tma-no-cluster": 2}[form])
    try:
        _decode_split_case(ops, g, dtype, hd, n_heads, n_kv, window)
    finally:
        decode_force_plain(False)
    assert decode_wait_timeouts() == 0


def _decode_split_case(ops, g, dtype, hd, n_heads, n_kv, window):
    lens = [700, 1, 64, 65, 130]
    table, kp, vp, ks, vs = make_cache(g, dtype, len(lens), lens, n_kv, hd)
    row_seq = torch.arange(len(lens), dtype=torch.int32)
    row_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    q = torch.randn(len(lens), n_heads * hd + 8, generator=g).to(DT[dtype])
    scale = 0.9 / math.sqrt(hd)
    ref = attention_ref(q[:, :n_heads * hd], ks, vs, row_seq, row_pos, n_heads, scale, window)
    q_d = dev(q)[:, :n_heads * hd]
    for splits in (1, 2, 5, 11):
        out = torch.full((len(lens), n_heads * hd), float("nan"), device="cuda", dtype=DT[dtype])
        scratch = torch.full((len(lens) * n_heads * splits * (hd + 2),), float("nan"), device="cuda")
        ops.attention_decode(q_d, out, dev(row_seq), dev(row_pos), dev(table), dev(kp), dev(vp), n_heads, scale, window,
                             n_splits=splits, scratch=scratch if splits > 1 else None)
        assert rel(out, ref) < KTOL[dtype], (splits,)
    with pytest.raises(KernelError, match="scratch"):
        ops.attention_decode(q_d, out, dev(row_seq), dev(row_pos), dev(table), dev(kp), dev(vp), n_heads, scale, window,
                             n_splits=3, scratch=None)
    # the step's own key and value handed in beside the cache: their place in the cache holds NaN before the
    # launch and the right rows after it, the result is the same, and the last CTA merges (twice: the counters
    # it uses must come back to zero)
    kw = n_kv * hd
    new = torch.zeros(len(lens), 2 * kw + 8).to(DT[dtype])
    kp2, vp2 = kp.clone(), vp.clone()
    for s_, l in enumerate(lens):
        new[s_, :kw], new[s_, kw:2 * kw] = ks[s_][l - 1].reshape(-1), vs[s_][l - 1].reshape(-1)
        kp2[table[s_, (l - 1) // 64], :, (l - 1) % 64] = float("nan")
        vp2[table[s_, (l - 1) // 64], :, (l - 1) % 64] = float("nan")
    new_d, kp_d, vp_d = dev(new), dev(kp2), dev(vp2)
    for splits in (1, 3, 3, 8, 16):
        out = torch.full((len(lens), n_heads * hd), float("nan"), device="cuda", dtype=DT[dtype])
        scratch = torch.full((len(lens) * n_heads * splits * (hd + 2),), float("nan"), device="cuda")
        ops.attention_decode(q_d, out, dev(row_seq), dev(row_pos), dev(table), kp_d, vp_d, n_heads, scale, window,
                             n_splits=splits, scratch=scratch, k_new=new_d[:, :kw], v_new=new_d[:, kw:2 * kw],
                             merge_in_kernel=True)
        assert rel(out, ref) < KTOL[dtype], ("new", splits)
        same = lambda a, b: torch.equal(torch.nan_to_num(a.float().cpu(), nan=7.0), torch.nan_to_num(b.float(), nan=7.0))
        assert same(kp_d, kp) and same(vp_d, vp)
    assert int(ops._counters.abs().sum()) == 0


@pytest.mark.parametrize("hd,n_heads,n_kv,window", [(64, 12, 12, 0), (128, 4, 2, 0), (32, 6, 3, 70), (16, 4, 4, 0)])
def test_attention_decode_from_sums_without_bias(hd, n_heads, n_kv, window):
    """Queries, keys and values handed in as 32-bit sums without their bias: the kernel adds the bias and rounds,
    so its result and what it writes to the cache equal, bit for bit, those of the same launch given the rounded
    rows; and it leaves the other buffer cleared."""
    from kvad_b200.ops import decode_wait_timeouts
    g = torch.Generator().manual_seed(31 * hd + n_heads)
    ops = Ops(torch.bfloat16)
    lens = [700, 1, 64, 65, 130]
    n = len(lens)
    table, kp, vp, ks, vs = make_cache(g, "bfloat16", n, lens, n_kv, hd)
    row_seq = torch.arange(n, dtype=torch.int32)
    row_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    qw, kw = n_heads * hd, n_kv * hd
    scale = 0.9 / math.sqrt(hd)
    sums = torch.randn(n, qw + 2 * kw, generator=g)
    for bias in (torch.randn(qw + 2 * kw, generator=g), torch.randn(qw + 2 * kw, generator=g).bfloat16(), None):
        rows = (sums + (bias.float() if bias is not None else 0)).bfloat16()            # what a storing product would have left
        buffers = torch.full((2, 16, qw + 2 * kw + 8), 3.0, device="cuda")
        buffers[0, :n, :qw + 2 * kw] = dev(sums)
        results = []
        for form in ("rows", "sums"):
            kp_d, vp_d = dev(kp), dev(vp)
            for s_, l in enumerate(lens):                      # the rows' own places hold NaN before the launch
                kp_d[table[s_, (l - 1) // 64], :, (l - 1) % 64] = float("nan")
                vp_d[table[s_, (l - 1) // 64], :, (l - 1) % 64] = float("nan")
            for splits in (1, 3, 6):
                out = torch.full((n, qw), float("nan"), device="cuda", dtype=torch.bfloat16)
                scratch = torch.full((n * n_heads * splits * (hd + 2),), float("nan"), device="cuda")
                if form == "rows":
                    r_d = dev(rows)
                    ops.attention_decode(r_d[:, :qw], out, dev(row_seq), dev(row_pos), dev(table), kp_d, vp_d, n_heads, scale, window,
                                         n_splits=splits, scratch=scratch, k_new=r_d[:, qw:qw + kw], v_new=r_d[:, qw + kw:],
                                         merge_in_kernel=True)
                else:
                    buffers[1].fill_(3.0)
                    ops.attention_decode_sums(buffers[0, :n, :qw + 2 * kw], None if bias is None else dev(bias), qw, qw + kw, buffers[1],
                                              out, dev(row_seq), dev(row_pos), dev(table), kp_d, vp_d, n_heads, scale, window,
                                              n_splits=splits, scratch=scratch)
                    assert float(buffers[1].abs().sum()) == 0.0
                results.append((out.float().cpu(), kp_d.float().cpu(), vp_d.float().cpu()))
        for a, b in zip(results[:3], results[3:]):                 # (places of the cache that no sequence uses hold NaN)
            assert all(torch.equal(torch.nan_to_num(x, nan=7.0), torch.nan_to_num(y, nan=7.0)) for x, y in zip(a, b))
        assert not torch.isnan(results[3][0]).any() and not torch.isnan(results[3][1][table[0, 699 // 64], :, 699 % 64]).any()
    assert decode_wait_timeouts() == 0
    assert int(ops._counters.abs().sum()) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,n_heads,n_kv,window", [(64, 12, 12, 0), (128, 8, 2, 0), (32, 10, 5, 100), (256, 12, 12, 0)])
def test_attention_decode_many_pairs(dtype, hd, n_heads, n_kv, window):
    """More (row, head) pairs than CTAs fit the GPU at once (the grid runs in waves), with sequences of very unequal
    length: what the reference gives, the same bits on a second launch, and the step's own keys and values taken
    from the projection's output and written to the cache."""
    from kvad_b200.ops import decode_force_plain, decode_wait_timeouts
    g = torch.Generator().manual_seed(11 * hd + n_heads)
    ops = Ops(DT[dtype])
    n_rows = 460 // n_heads + 3
    lens = [int(x) for x in torch.randint(1, 330, (n_rows,), generator=g)]
    lens[0], lens[1], lens[2] = 1, 64, 65
    table, kp, vp, ks, vs = make_cache(g, dtype, n_rows, lens, n_kv, hd)
    row_seq = torch.arange(n_rows, dtype=torch.int32)
    row_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32)
    q = torch.randn(n_rows, n_heads * hd, generator=g).to(DT[dtype])
    scale = 0.9 / math.sqrt(hd)
    ref = attention_ref(q, ks, vs, row_seq, row_pos, n_heads, scale, window)
    outs = []
    for mode in (0, 0):
        decode_force_plain(mode)
        try:
            out = torch.full((n_rows, n_heads * hd), float("nan"), device="cuda", dtype=DT[dtype])
            ops.attention_decode(dev(q), out, dev(row_seq), dev(row_pos), dev(table), dev(kp), dev(vp), n_heads, scale, window)
        finally:
            decode_force_plain(0)
        assert rel(out, ref) < KTOL[dtype], mode
        outs.append(out)
    assert torch.equal(outs[0], outs[1])             # the same bits every time
    # with the step's own keys and values handed in (and written to the cache by the kernel)
    kn = torch.stack([ks[s][l - 1].reshape(-1) for s, l in enumerate(lens)]).to(DT[dtype])
    vn = torch.stack([vs[s][l - 1].reshape(-1) for s, l in enumerate(lens)]).to(DT[dtype])
    kp2, vp2 = kp.clone(), vp.clone()
    for s, l in enumerate(lens):
        kp2[table[s, (l - 1) // 64], :, (l - 1) % 64] = float("nan")
        vp2[table[s, (l - 1) // 64], :, (l - 1) % 64] = float("nan")
    kp_d, vp_d = dev(kp2), dev(vp2)
    new = torch.cat([kn, vn], dim=1).cuda()
    w = n_kv * hd
    out = torch.full((n_rows, n_heads * hd), float("nan"), device="cuda", dtype=DT[dtype])
    ops.attention_decode(dev(q), out, dev(row_seq), dev(row_pos), dev(table), kp_d, vp_d, n_heads, scale, window,
                         k_new=new[:, :w], v_new=new[:, w:])
    assert rel(out, ref) < KTOL[dtype]
    same = lambda a, b: torch.equal(torch.nan_to_num(a.float().cpu(), nan=7.0), torch.nan_to_num(b.float(), nan=7.0))
    assert same(kp_d, kp) and same(vp_d, vp)
    assert decode_wait_timeouts() == 0


def test_attention_decode_finds_one_far_key():
    g = torch.Generator().manual_seed(19)
    ops = Ops(torch.bfloat16)
    hd, n = 64, 1000
    table, kp, vp, ks, vs = make_cache(g, "bfloat16", 1, [n], 1, hd)
    far = 70
    q = torch.randn(1, hd, generator=g).bfloat16()
    ks[0][far, 0] = (q[0].float() * 30.0 / q[0].float().pow(2).sum()).bfloat16()
    ks[0][:, 0][torch.arange(n) != far] *= 0.05
    vs[0][far, 0] = torch.arange(hd).bfloat16()
    table, kp, vp, _, _ = rebuild(table, kp, vp, ks, vs)
    row_seq, row_pos = torch.zeros(1, dtype=torch.int32), torch.tensor([n - 1], dtype=torch.int32)
    for splits in (1, 4, 16):
        out = torch.empty(1, hd, device="cuda", dtype=torch.bfloat16)
        scratch = torch.empty(splits * (hd + 2), device="cuda")
        ops.attention_decode(dev(q), out, dev(row_seq), dev(row_pos), dev(table), dev(kp), dev(vp), 1, 1.0, 0,
                             n_splits=splits, scratch=scratch)
        assert (out.float().cpu()[0] - torch.arange(hd)).abs().max() < 0.05 * hd
    assert not ops.decode_takes(144) and ops.decode_takes(96)


@pytest.mark.parametrize("hd,n_heads,n_kv,window", [(16, 4, 4, 0), (32, 3, 3, 0), (48, 6, 2, 0), (64, 12, 12, 0), (80, 3, 1, 0),
                                                    (96, 2, 2, 0), (112, 2, 1, 0), (128, 2, 2, 50), (64, 4, 2, 70), (32, 5, 5, 64)])
@pytest.mark.parametrize("form", ["auto", "mma.sync", "split"])
def test_attention_prefill_tensor_cores(hd, n_heads, n_kv, window, form):
    """Whole prompts, prompts that continue cached positions, a single row and a row count that is no multiple
    of the tile, in one launch; the pages hold NaN wherever no position lies.  Head sizes 64 and 128 run on
    tcgen05 unless the older mma.sync kernel is forced.  "split": every tile of rows that sees two pages or more is
    walked by both slots of its CTA, half of the pages each (by itself the kernel does that from nine pages on)."""
    from kvad_b200.ops import prefill_force_legacy, prefill_split_above, prefill_wait_timeouts
    if form != "auto" and hd not in (64, 128):
        pytest.skip("this head size has one kernel only")
    prefill_force_legacy(form == "mma.sync")
    prefill_split_above(1 if form == "split" else 0)
    try:
        _attention_prefill_case(hd, n_heads, n_kv, window)
    finally:
        prefill_force_legacy(False)
        prefill_split_above(0)
    assert prefill_wait_timeouts() == 0


def _attention_prefill_case(hd, n_heads, n_kv, window):
    g = torch.Generator().manual_seed(3 * hd + n_heads + window)
    ops = Ops(torch.bfloat16)
    lens = [200, 1, 64, 65, 300, 130, 650]            # lengths after the step
    new = [200, 1, 64, 65, 37, 129, 600]              # rows the step brings (the rest was cached before)
    table, kp, vp, ks, vs = make_cache(g, "bfloat16", len(lens), lens, n_kv, hd)
    rows = [(s, p) for s, (l, n) in enumerate(zip(lens, new)) for p in range(l - n, l)]
    row_seq = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    row_pos = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    seq_starts = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32)
    kv_lens = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(len(rows), n_heads * hd + 8, generator=g).bfloat16()
    scale = 0.8 / math.sqrt(hd)
    ref = attention_ref(q[:, :n_heads * hd], ks, vs, row_seq, row_pos, n_heads, scale, window)
    out = torch.full((len(rows), n_heads * hd), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops.attention_prefill(dev(q)[:, :n_heads * hd], out, dev(seq_starts), dev(kv_lens), len(lens), max(new), dev(table),
                          dev(kp), dev(vp), n_heads, scale, window)
    assert rel(out, ref) < KTOL["bfloat16"]
    # the general kernel agrees on the same launch
    out2 = torch.full_like(out, float("nan"))
    ops.attention(dev(q)[:, :n_heads * hd], out2, dev(row_seq), dev(row_pos), dev(table), dev(kp), dev(vp), n_heads, scale, window)
    assert rel(out2, ref) < KTOL["bfloat16"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("hd,n_heads,n_kv,window", [(16, 4, 4, 0), (48, 6, 2, 0), (64, 12, 12, 0), (80, 3, 1, 70), (128, 2, 2, 50),
                                                    (256, 2, 1, 0), (20, 2, 2, 0), (36, 3, 3, 9)])
def test_attention_prompt_tiled_on_cuda_cores(dtype, hd, n_heads, n_kv, window):
    """The tiled CUDA-core kernel for prompts (the float32 engine's; in bfloat16 what the tensor-core kernel refuses):
    whole prompts, prompts that continue cached positions, a single row, row counts that are no multiple of its 32
    rows, windows that end inside a page; the pages hold NaN wherever no position lies."""
    g = torch.Generator().manual_seed(5 * hd + n_heads + window)
    ops = Ops(DT[dtype])
    lens = [200, 1, 64, 65, 300, 130, 650]            # lengths after the step
    new = [200, 1, 64, 65, 37, 129, 600]              # rows the step brings (the rest was cached before)
    table, kp, vp, ks, vs = make_cache(g, dtype, len(lens), lens, n_kv, hd)
    rows = [(s, p) for s, (l, n) in enumerate(zip(lens, new)) for p in range(l - n, l)]
    row_seq = torch.tensor([r[0] for r in rows], dtype=torch.int32)
    row_pos = torch.tensor([r[1] for r in rows], dtype=torch.int32)
    seq_starts = torch.tensor([0] + list(np.cumsum(new)), dtype=torch.int32)
    kv_lens = torch.tensor(lens, dtype=torch.int32)
    q = torch.randn(len(rows), n_heads * hd + 8, generator=g).to(DT[dtype])
    scale = 0.8 / math.sqrt(hd)
    ref = attention_ref(q[:, :n_heads * hd], ks, vs, row_seq, row_pos, n_heads, scale, window)
    assert ops.prompt_takes(hd, 64) and not ops.prompt_takes(hd, 32) and not ops.prompt_takes(260, 64) and not ops.prompt_takes(18, 64)
    out = torch.full((len(rows), n_heads * hd), float("nan"), device="cuda", dtype=DT[dtype])
    ops.attention_prompt(dev(q)[:, :n_heads * hd], out, dev(seq_starts), dev(kv_lens), len(lens), max(new), dev(table),
                         dev(kp), dev(vp), n_heads, scale, window)
    assert rel(out, ref) < KTOL[dtype]
    # the row-by-row kernel agrees (to rounding in 32-bit: another order of additions)
    out2 = torch.full_like(out, float("nan"))
    ops.attention(dev(q)[:, :n_heads * hd], out2, dev(row_seq), dev(row_pos), dev(table), dev(kp), dev(vp), n_heads, scale, window)
    assert rel(out2, out.float().cpu()) < (1e-5 if dtype == "float32" else KTOL[dtype])


def test_attention_prefill_finds_one_far_key():
    g = torch.Generator().manual_seed(29)
    ops = Ops(torch.bfloat16)
    hd, n = 64, 900
    table, kp, vp, ks, vs = make_cache(g, "bfloat16", 1, [n], 1, hd)
    far = 5
    q = torch.randn(n, hd, generator=g).bfloat16() * 0.1
    q[n - 1] = torch.randn(hd, generator=g).bfloat16()
    ks[0][far, 0] = (q[n - 1].float() * 30.0 / q[n - 1].float().pow(2).sum()).bfloat16()
    ks[0][:, 0][torch.arange(n) != far] *= 0.05
    vs[0][far, 0] = torch.arange(hd).bfloat16()
    table, kp, vp, _, _ = rebuild(table, kp, vp, ks, vs)
    out = torch.empty(n, hd, device="cuda", dtype=torch.bfloat16)
    ops.attention_prefill(dev(q), out, dev(torch.tensor([0, n], dtype=torch.int32)), dev(torch.tensor([n], dtype=torch.int32)),
                          1, n, dev(table), dev(kp), dev(vp), 1, 1.0, 0)
    assert (out.float().cpu()[n - 1] - torch.arange(hd)).abs().max() < 0.05 * hd
    assert not ops.prefill_takes(256) and not ops.prefill_takes(24)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
@pytest.mark.parametrize("m", [1, 2, 3, 4, 7, 8, 13, 16])
def test_linear_weight_streaming_form(m, dtype):
    """At most 16 rows: a warp per output column, the column's weights held in registers; bfloat16 and true 32-bit."""
    ops = Ops(DT[dtype])
    g = torch.Generator().manual_seed(400 + m)
    shapes = [(768, 768), (1000, 96), (50, 320), (2304, 64), (777, 3072), (50257, 768), (333, 1600), (40, 4096), (24, 6400), (9, 8)]
    if dtype == "float32":
        shapes = [(n, k) for n, k in shapes if k <= 4096 and max(1, 1 << (m - 1).bit_length()) * k * 4 <= 200 * 1024] + [(31, 12)]
    for n, k in shapes:
        for epi in ("store", "gelu_tanh", "gelu_erf", "residual", "store_f32"):
            assert linear_case(ops, dtype, m, n, k, epi, g, form="rows") < KTOL[dtype], (m, n, k, epi)
    assert linear_case(ops, dtype, m, 333, 128, "store", g, bias=False, strided=True, form="rows") < KTOL[dtype]
    assert linear_case(ops, dtype, m, 333, 128, "residual", g, bias_f32=True, form="rows") < KTOL[dtype]
    with pytest.raises(KernelError, match="at most 16 rows"):
        linear_case(ops, dtype, 17, 64, 64, "store", g, form="rows")


def test_a_bounded_wait_that_runs_out_is_reported_and_harmless():
    """A load that never comes: the launch's wait for it runs out after the (shortened) limit, the status counter
    says so, the launch frees what it holds and returns - and the next, ordinary launch is right.  Nothing here
    faults or hangs: the kernel is told to leave out one load, and its wait gives up by counting."""
    from kvad_b200.ops import tcgen05_test_hooks, tcgen05_wait_timeouts
    ops = Ops(torch.bfloat16)
    if not ops.tensor_core_linear:
        pytest.skip("no tensor-core linear kernel")
    g = torch.Generator().manual_seed(9)
    assert linear_case(ops, "bfloat16", 32, 128, 128, "store", g, form="swapped") < KTOL["bfloat16"]
    before = tcgen05_wait_timeouts()
    a = dev(torch.randn(32, 128, generator=g).bfloat16())
    w = dev((torch.randn(128, 128, generator=g) / 11).bfloat16())
    out = torch.zeros(32, 128, device="cuda", dtype=torch.bfloat16)
    try:
        tcgen05_test_hooks(wait_limit=4096, skip_first_load=True)
        ops.linear(a, w, None, out, "store", form="swapped")          # one CTA; stage 0 is never filled
        torch.cuda.synchronize()                                       # returns: no hang
        assert tcgen05_wait_timeouts() > before
    finally:
        tcgen05_test_hooks(0, False)
    again = tcgen05_wait_timeouts()
    assert linear_case(ops, "bfloat16", 32, 128, 128, "store", g, form="swapped") < KTOL["bfloat16"]
    assert linear_case(ops, "bfloat16", 300, 200, 256, "gelu_tanh", g) < KTOL["bfloat16"]
    assert tcgen05_wait_timeouts() == again
