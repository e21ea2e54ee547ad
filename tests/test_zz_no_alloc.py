"""The allocation-free decode attention, called the way its users call it: through the exported C
symbol of the compiled library, with raw pointers.

Those users are hosts without an allocator to lend: a program that links only this kernel library,
a plug-in inside an application that owns all device memory, a loop that cannot afford cudaMalloc.
The entry point keeps its scratch in a device array of the library itself; this test checks that
its output is the ordinary entry point's, on two calls in a row (the second finds the array as the
first left it), that sizes beyond the array are refused, and that no device memory is allocated
by the calls.  It runs last so that a run that stops at the first failure has seen every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_int64, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

SCRATCH_FLOATS = 1 << 20


def entry_points():
    from kvad_b200.csrc import build

    lib = build.load("attention_decode")
    args = [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
    tail = [c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p]
    noalloc = lib.kvad_attention_decode_noalloc
    noalloc.argtypes, noalloc.restype = args + tail, c_int
    plain = lib.kvad_attention_decode
    plain.argtypes, plain.restype = args + [c_void_p] + tail, c_int
    need = lib.kvad_attention_decode_noalloc_need
    need.argtypes, need.restype = [c_int, c_int, c_int, c_int], c_int64
    return lib, noalloc, plain, need


def make_case(seed, n_seqs, n_heads, n_kv, hd, lens):
    g = torch.Generator().manual_seed(seed)
    pages_per = [-(-l // 64) for l in lens]
    n_pages = sum(pages_per) + 2
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros((n_seqs, max(pages_per)), dtype=torch.int32)
    it = iter(order)
    for s, n in enumerate(pages_per):
        for p in range(n):
            table[s, p] = next(it)
    kp = torch.randn(n_pages, n_kv, 64, hd, generator=g).bfloat16().cuda()
    vp = torch.randn(n_pages, n_kv, 64, hd, generator=g).bfloat16().cuda()
    q = torch.randn(n_seqs, n_heads * hd, generator=g).bfloat16().cuda()
    row_seq = torch.arange(n_seqs, dtype=torch.int32).cuda()
    row_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32).cuda()
    return q, table.cuda(), kp, vp, row_seq, row_pos


def test_no_alloc_entry_point_matches_the_ordinary_one_twice():
    lib, noalloc, plain, need = entry_points()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    n_heads, n_kv, hd = 6, 2, 64
    for call, (lens, splits) in enumerate([([700, 1, 64, 65, 130], 5), ([300, 513, 90], 8)]):
        q, table, kp, vp, row_seq, row_pos = make_case(100 + call, len(lens), n_heads, n_kv, hd, lens)
        n = len(lens)
        scale = 1.0 / math.sqrt(hd)
        want = torch.full((n, n_heads * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty(n * n_heads * splits * (hd + 2), dtype=torch.float32, device="cuda")
        rc = plain(1, q.data_ptr(), q.stride(0), want.data_ptr(), want.stride(0), row_seq.data_ptr(), row_pos.data_ptr(),
                   table.data_ptr(), table.shape[1], kp.data_ptr(), vp.data_ptr(), scratch.data_ptr(), n, n_heads, n_kv,
                   hd, 64, splits, scale, 0, stream)
        assert rc == 0, lib.kvad_last_error().decode()
        got = torch.full_like(want, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.mem_get_info()[0]
        rc = noalloc(1, q.data_ptr(), q.stride(0), got.data_ptr(), got.stride(0), row_seq.data_ptr(), row_pos.data_ptr(),
                     table.data_ptr(), table.shape[1], kp.data_ptr(), vp.data_ptr(), n, n_heads, n_kv, hd, 64, splits,
                     scale, 0, stream)
        assert rc == 0, lib.kvad_last_error().decode()
        torch.cuda.synchronize()
        if call == 1:                       # the first call may have brought the library's own data in
            assert torch.cuda.mem_get_info()[0] >= before, "the call allocated device memory"
        assert need(n, n_heads, hd, splits) == n * n_heads * splits * (hd + 2)
        assert torch.isfinite(got.float()).all()
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 6e-3 * want.float().abs().max().item(), (call, diff)
        assert torch.equal(got, want)       # same kernel, same splits: the same bits


def test_no_alloc_entry_point_refuses_what_its_array_cannot_hold():
    lib, noalloc, plain, need = entry_points()
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    q, table, kp, vp, row_seq, row_pos = make_case(7, 2, 4, 4, 64, [100, 200])
    out = torch.empty_like(q)
    # 4096 rows x 64 heads x 16 splits x 66 floats is far beyond 2^20
    assert need(4096, 64, 64, 16) > SCRATCH_FLOATS
    rc = noalloc(1, q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), row_seq.data_ptr(), row_pos.data_ptr(),
                 table.data_ptr(), table.shape[1], kp.data_ptr(), vp.data_ptr(), 4096, 64, 64, 64, 64, 16, 0.125, 0, stream)
    assert rc != 0
    msg = lib.kvad_last_error().decode()
    assert "exceed the built-in" in msg and "1048576" in msg
    # one split needs no scratch at all and is served whatever the sizes
    rc = noalloc(1, q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0), row_seq.data_ptr(), row_pos.data_ptr(),
                 table.data_ptr(), table.shape[1], kp.data_ptr(), vp.data_ptr(), 2, 4, 4, 64, 64, 1, 0.125, 0, stream)
    assert rc == 0, lib.kvad_last_error().decode()
    torch.cuda.synchronize()
    assert torch.isfinite(out.float()).all()
