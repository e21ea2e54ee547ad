"""Python face of the CUDA kernels.

One `Ops` object serves one compute dtype (float32 or bfloat16).  Its methods
check what the kernels assume (device, dtype, contiguity, sizes), pass raw
pointers and the current CUDA stream to the C entry points, and raise
`KernelError` with the kernel's own message when an entry point refuses.
Tensors are torch tensors only as owners of device memory; no torch operator
computes anything here, and nothing falls back to the CPU.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from .csrc import build

F32, BF16 = 0, 1
EPILOGUES = {"store": 0, "gelu_tanh": 1, "gelu_erf": 2, "residual": 3, "store_f32": 4}


class KernelError(RuntimeError):
    pass


def _code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kvad_b200 kernels compute in float32 or bfloat16, not {dtype}")


def _ptr(t: Optional[torch.Tensor]):
    return c_void_p(0 if t is None else t.data_ptr())


_SIGNATURES = {
    "rows": {
        "kvad_embed": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
        "kvad_layernorm": [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_void_p],
        "kvad_kv_store": [c_int, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                          c_int, c_int, c_int, c_int, c_void_p],
        "kvad_zero_bytes": [c_void_p, c_int64, c_void_p],
    },
    "linear_simt": {
        "kvad_linear_simt": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int,
                             c_int, c_void_p],
    },
    "linear_tcgen05": {
        "kvad_linear_tcgen05": [c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int,
                                c_int, c_int, c_void_p],
        "kvad_linear_tcgen05_status": [],
    },
    "linear_rows": {
        "kvad_linear_rows": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                             c_void_p],
    },
    "linear_rows_f32": {
        "kvad_linear_rows": [c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_int, c_int, c_int,
                             c_void_p],
    },
    "attention_simt": {
        "kvad_attention_simt": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "kvad_attention_tiled": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
    },
    "attention_prefill": {
        "kvad_attention_prefill": [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                   c_void_p, c_void_p, c_int64, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int,
                                   c_void_p],
    },
    "attention_decode": {
        "kvad_attention_decode_step": [c_int, c_void_p, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int,
                                       c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int,
                                       c_int, c_int, c_int, c_int, c_float, c_int, c_void_p],
        "kvad_attention_decode_pre": [c_void_p, c_int64, c_void_p, c_int, c_int, c_int, c_void_p, c_int64],
        "kvad_attention_decode_takes_pre": [c_int, c_int, c_int],
    },
    "sampling": {
        "kvad_sample": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
        "kvad_argmax": [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p],
    },
}

_bound: dict[str, ctypes.CDLL] = {}
_pdl = os.environ.get("KVAD_PDL", "1") != "0"
_switch_epoch = 0          # bumped by every switch that changes which kernels a step launches


def register_kernels(name: str, source: str, signatures: dict) -> None:
    """The door for a part that brings a kernel of its own: `source` is a `.cu` file anywhere (it may
    include this package's `common.cuh`; it must contain `KVAD_DEFINE_LAST_ERROR()` once), `signatures`
    maps its exported C entry points (returning 0 or a negative code, message through
    `kvad_last_error`) to their ctypes argument lists.  Afterwards `lib(name)` compiles it for
    sm_100a on first use and loads it like the package's own libraries; `launch(handle, status)`
    turns a refusal into a `KernelError` and counts the launch."""
    if name in _SIGNATURES and name not in build.registered_sources():
        raise ValueError(f"`{name}` is one of the package's own kernel libraries")
    build.register_source(name, source)
    _SIGNATURES[name] = dict(signatures)
    _bound.pop(name, None)


def switches_changed() -> None:
    """Called by every switch that changes which kernels a step launches: captured step graphs are
    keyed by the epoch, so a step captured under the old setting is not replayed under the new one."""
    global _switch_epoch
    _switch_epoch += 1


def switch_epoch() -> int:
    return _switch_epoch


def set_pdl(on: bool) -> None:
    """Programmatic dependent launch for every kernel of the library: a kernel may start (set up,
    fetch its weights) while the one before it in the stream still runs.  On by default; KVAD_PDL=0
    or set_pdl(False) launches plainly."""
    global _pdl
    _pdl = bool(on)
    switches_changed()
    for handle in _bound.values():
        handle.kvad_set_pdl(int(_pdl))


def lib(name: str) -> ctypes.CDLL:
    """The loaded kernel library `name` with its entry points typed."""
    hit = _bound.get(name)
    if hit is not None:
        return hit
    handle = build.load(name)
    for fn, argtypes in _SIGNATURES[name].items():
        f = getattr(handle, fn)
        f.argtypes = argtypes
        f.restype = c_int
    handle.kvad_set_pdl.argtypes = [c_int]
    handle.kvad_set_pdl.restype = None
    handle.kvad_set_pdl(int(_pdl))
    _bound[name] = handle
    return handle


def libraries_for(dtype: torch.dtype) -> list[str]:
    """Which kernel libraries a model of this compute dtype loads."""
    names = ["rows", "linear_simt", "attention_simt", "sampling"]
    names += [n for n in ("linear_rows" if dtype == torch.bfloat16 else "linear_rows_f32", "attention_decode") if n in build.sources()]
    if dtype == torch.bfloat16:
        names += [n for n in ("linear_tcgen05", "attention_prefill") if n in build.sources()]
    return names


_launches = 0


def launch_count() -> int:
    """How many kernels of this library have been launched (or captured into a graph) so far."""
    return _launches


def launch(handle: ctypes.CDLL, status: int) -> None:
    """For kernels registered from outside: raises the entry point's own message on a refusal, counts the launch."""
    _check(status, handle)


def stream_ptr() -> c_void_p:
    """The current CUDA stream as the entry points take it."""
    return _stream()


_sm_counts: dict[int, int] = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device)."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    n = _sm_counts.get(idx)
    if n is None:
        n = _sm_counts[idx] = int(torch.cuda.get_device_properties(idx).multi_processor_count)
    return n


def _check(status: int, handle: ctypes.CDLL) -> None:
    global _launches
    if status != 0:
        raise KernelError(handle.kvad_last_error().decode("utf-8", "replace"))
    _launches += 1


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kvad_b200 kernels run on CUDA tensors only; there is no CPU path")


def _rows_view(t: torch.Tensor, what: str) -> int:
    """Leading dimension of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{what}: needs a 2-D tensor with contiguous rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


class Ops:
    """Kernels bound to one compute dtype."""

    def __init__(self, dtype: torch.dtype):
        self.dtype = dtype
        self.code = _code(dtype)
        self.use_tensor_cores = dtype == torch.bfloat16
        # set to False to keep the bfloat16 engine on the CUDA-core kernels (tests compare both)
        self.tensor_core_linear = dtype == torch.bfloat16 and "linear_tcgen05" in build.sources()
        self.tensor_core_prefill = dtype == torch.bfloat16 and "attention_prefill" in build.sources()
        self.fast_decode = "attention_decode" in build.sources()        # both dtypes: the decode kernel is templated on the storage type
        # Up to 16 rows the product can also run as a stream of weights through registers on the CUDA cores
        # (linear_rows.cu).  Measured on a B200 it beats the tensor-core kernel at one or two rows (qkv at 1 row:
        # 2.4 us against 3.9 us; a GPT-2 small decode step at batch 1: 0.286 ms against 0.326 ms, at batch 2: 0.314
        # against 0.319) and loses from 4 rows on (batch 4: 0.410 ms against 0.327), and it loses on the output head
        # (50257 outputs: the step is 0.307 ms with it, 0.286 without).  So it takes products of at most
        # `rows_linear_max` rows and `ROWS_LINEAR_MAX_OUT` outputs; form="rows" selects it for any count up to 16.
        # In 32-bit there are no tensor cores to lose to: the weight stream is the decode road of the float32 engine
        # for every row count it takes (the tiled CUDA-core kernel would run one row in a tile of 64).
        self._rows_lib = "linear_rows" if dtype == torch.bfloat16 else "linear_rows_f32"     # one library per element type
        self.rows_linear_max = (2 if dtype == torch.bfloat16 else 16) if self._rows_lib in build.sources() else 0
        self.tiled_prompt = True    # prompts that the tensor-core kernel does not take: the tiled CUDA-core kernel, not the row-by-row one
        self._counters = None       # zeroed ints the decode kernel counts finished splits in (left zeroed by it)
        # Two 32-bit buffers [16, width] that q/k/v products of 3..16 rows add their shares of K into (see
        # `linear_sums`); they alternate call by call, and the kernel that reads one clears the other.
        self.qkv_sums = os.environ.get("KVAD_QKV_SUMS", "1") != "0"
        self._sums: Optional[torch.Tensor] = None
        self._sum_calls = 0
        self._sums_open = False         # between a step's first `linear_sums` and its `end_step`
        from . import profile
        if profile.enabled():       # KVAD_PROFILE=1: a table of device time per operation at exit
            profile.instrument(self)

    def path_key(self) -> tuple:
        """Everything on the host that decides which kernels a step of a given shape launches; part of
        the key under which a step's CUDA graph is kept."""
        return (_switch_epoch, self.tensor_core_linear, self.tensor_core_prefill, self.fast_decode,
                self.rows_linear_max, self.qkv_sums, self.SUMS_MIN_K, self.tiled_prompt)

    def begin_step(self) -> None:
        """Called once before a step's first kernel (inside the capture, if the step is being captured)."""
        if self._sums_open and self._sums is not None and not torch.cuda.is_current_stream_capturing():
            self._sums.zero_()              # a step before this one was given up half-way: start clean
        self._sum_calls = 0
        self._sums_open = False

    def end_step(self) -> None:
        """Called once after a step's last kernel.  The two buffers of `linear_sums` alternate and every reader clears
        the one it does not read, so after an even number of such products the first buffer is clean for the next
        step; after an odd number it is cleared here."""
        if self._sum_calls % 2 == 1:
            h = lib("rows")
            _check(h.kvad_zero_bytes(_ptr(self._sums), self._sums[0].numel() * 4, _stream()), h)
        self._sums_open = False

    # -- embedding -----------------------------------------------------------------
    def embed(self, tokens, positions, wte, wpe, out) -> None:
        _need_cuda(tokens, positions, wte, wpe, out)
        n, width = out.shape
        if wte.dtype != self.dtype or (wpe is not None and wpe.dtype != self.dtype):
            raise KernelError(f"embed: tables must be {self.dtype}")
        if out.dtype != torch.float32 or not out.is_contiguous() or wte.shape[1] != width:
            raise KernelError("embed: output must be contiguous float32 of the tables' width")
        if tokens.dtype != torch.int32 or tokens.numel() < n:
            raise KernelError("embed: tokens must be int32, one per row")
        h = lib("rows")
        _check(h.kvad_embed(self.code, _ptr(tokens), _ptr(positions), _ptr(wte), _ptr(wpe), _ptr(out), n, width,
                            wte.shape[0], 0 if wpe is None else wpe.shape[0], _stream()), h)

    # -- norms ---------------------------------------------------------------------
    def layernorm(self, x, gain, bias, eps: float, out, rows=None) -> None:
        _need_cuda(x, gain, bias, out, rows)
        n, width = out.shape
        if x.dtype != torch.float32 or not x.is_contiguous() or x.shape[1] != width:
            raise KernelError("layernorm: input must be the contiguous float32 residual stream")
        if out.dtype != self.dtype or not out.is_contiguous():
            raise KernelError(f"layernorm: output must be contiguous {self.dtype}")
        if gain.numel() != width or (bias is not None and (bias.numel() != width or bias.dtype != gain.dtype)):
            raise KernelError("layernorm: gain and bias must have the row's width and one dtype")
        if rows is None and x.shape[0] < n:
            raise KernelError("layernorm: fewer input rows than output rows")
        if rows is not None and (rows.dtype != torch.int32 or rows.numel() < n):
            raise KernelError("layernorm: row list must be int32, one per output row")
        params_f32 = 1 if gain.dtype == torch.float32 else 0
        if not params_f32 and gain.dtype != torch.bfloat16:
            raise KernelError(f"layernorm: gain must be float32 or bfloat16, not {gain.dtype}")
        h = lib("rows")
        _check(h.kvad_layernorm(self.code, _ptr(x), _ptr(rows), _ptr(gain), _ptr(bias), params_f32, _ptr(out), n, width,
                                float(eps), _stream()), h)

    # -- linear --------------------------------------------------------------------
    ROWS_LINEAR_MAX_OUT = 8192
    ROWS_BLOCKS_MAX = 64           # 32-bit: up to so many rows go through the weight-streaming form in blocks of 16

    def linear(self, a, weight, bias, out, epilogue: str = "store", *, tile: int = 0, splits: int = 0,
               form: str = "auto") -> None:
        """out = epilogue(a . weight^T + bias); weight is [out_features, in_features].

        `form`: "auto"; "rows" (at most 16 rows: weights streamed through registers on the CUDA cores);
        "wide" / "swapped" (the tensor-core kernel's two operand roles).  `tile` and `splits` fix the
        tensor-core kernel's tile width and K split (0: its own choice)."""
        _need_cuda(a, weight, bias, out)
        epi = EPILOGUES[epilogue]
        lda, ldo = _rows_view(a, "linear input"), _rows_view(out, "linear output")
        m, k = a.shape
        n = weight.shape[0]
        if weight.dim() != 2 or weight.shape[1] != k or not weight.is_contiguous():
            raise KernelError(f"linear: weight {tuple(weight.shape)} does not take inputs of width {k}")
        if a.dtype != self.dtype or weight.dtype != self.dtype:
            raise KernelError(f"linear: input and weight must be {self.dtype}")
        want_out = torch.float32 if epi >= 3 else self.dtype
        if out.dtype != want_out or out.shape[0] != m or out.shape[1] != n:
            raise KernelError(f"linear: output must be {want_out} of shape [{m}, {n}]")
        bias_f32 = 0
        if bias is not None:
            if bias.numel() != n:
                raise KernelError(f"linear: bias has {bias.numel()} entries for {n} outputs")
            bias_f32 = 1 if bias.dtype == torch.float32 else 0
            if not bias_f32 and bias.dtype != torch.bfloat16:
                raise KernelError(f"linear: bias must be float32 or bfloat16, not {bias.dtype}")
        ve = 8 if self.dtype == torch.bfloat16 else 4          # elements of a 16-byte piece
        # (beyond ROWS_LINEAR_MAX_OUT outputs - the head - the tensor-core form is as fast or faster, except for one row
        # of long K: 50257 x 1600 at one row 26 us against 44)
        rows_out_ok = self.dtype == torch.float32 or n <= self.ROWS_LINEAR_MAX_OUT or (m == 1 and k >= 1536)
        # (by itself only up to K = 4096: beyond, one column a warp is too long a chain - measured at 1600 x 6400,
        # one row: the tensor-core form with K split over twelve CTAs is 10 % faster on the step)
        # (three and four rows too where the product STORES and K is short - there the tensor-core form needs a cluster:
        # at GPT-2 small's sizes a step of 3 or 4 sequences 0.320 -> 0.301 ms; at K = 1024 and 1600 it loses 1..6 %)
        rows_auto = m <= self.rows_linear_max or (m <= self.rows_linear_max + 2 and epi < 3 and k <= 768 and self.dtype == torch.bfloat16)
        if ((form == "rows" or (form == "auto" and rows_auto and rows_out_ok and k <= 4096)) and m <= 16 and k <= 1024 * ve
                and k % ve == 0 and lda % ve == 0 and (1 << max(0, m - 1).bit_length()) * k * a.element_size() <= 200 * 1024
                and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and self._rows_lib in build.sources()):
            h = lib(self._rows_lib)
            _check(h.kvad_linear_rows(self.code, _ptr(a), lda, _ptr(weight), _ptr(bias), bias_f32, _ptr(out), ldo, m, n, k, epi,
                                      _stream()), h)
            return
        if form == "rows":
            raise KernelError("linear: the weight-streaming form takes at most 16 rows and K a multiple of a 16-byte piece, at most 1024 pieces")
        if (form == "auto" and self.dtype == torch.float32 and self.rows_linear_max >= 16 and 16 < m <= self.ROWS_BLOCKS_MAX and k <= 4096
                and k % ve == 0 and lda % ve == 0 and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0 and self._rows_lib in build.sources()):
            # 32-bit, 17..64 rows: the tiled kernel would run a grid of N / 64 CTAs, each walking all of K (17 rows of
            # 768 x 3072: 265 us); the weight-streaming form takes the rows in blocks of up to 16 instead, the later
            # blocks finding the weights in the L2 (a decode step of 17 sequences at GPT-2 small's sizes: 6.1 -> 1.0 ms, of 64: 2.9)
            block = 16
            while block > 1 and block * k * 4 > 200 * 1024:
                block //= 2
            h = lib(self._rows_lib)
            for m0 in range(0, m, block):
                rows = min(block, m - m0)
                _check(h.kvad_linear_rows(self.code, c_void_p(a.data_ptr() + m0 * lda * 4), lda, _ptr(weight), _ptr(bias), bias_f32,
                                          c_void_p(out.data_ptr() + m0 * ldo * 4), ldo, rows, n, k, epi, _stream()), h)
            return
        if self.tensor_core_linear and tcgen05_takes(a, weight, out, lda, ldo):
            h = lib("linear_tcgen05")
            force = (int(tile) & 0xffff) | ((int(splits) & 0xff) << 16) | ({"auto": 0, "wide": 1, "swapped": 2}.get(form, 0) << 24)
            _check(h.kvad_linear_tcgen05(_ptr(a), lda, _ptr(weight), _ptr(bias), bias_f32, _ptr(out), ldo, m, n, k,
                                         epi, force, _stream()), h)
            return
        h = lib("linear_simt")
        _check(h.kvad_linear_simt(self.code, _ptr(a), lda, _ptr(weight), _ptr(bias), bias_f32, _ptr(out), ldo, m, n, k,
                                  epi, _stream()), h)

    SUMS_MIN_K = 1536

    def sums_take(self, m: int, weight, head_dim: int, page_size: int) -> bool:
        """Whether a q/k/v product of `m` rows leaves 32-bit sums for the decode attention to finish (see `linear_sums`).
        Only where K is long (from 1536 on): there the cluster of the storing form costs most (GPT-2 XL's sizes, 8
        rows: +4 % on the step); at K = 768 the two forms are even (+0.8 %) and at K = 1024 this one loses (-1.8 %)."""
        n, k = weight.shape
        return bool(self.qkv_sums and self.dtype == torch.bfloat16 and self.rows_linear_max < m <= 16 and self.tensor_core_linear
                    and self.fast_decode and k % 64 == 0 and k >= self.SUMS_MIN_K and n % 8 == 0 and weight.data_ptr() % 16 == 0 and "linear_tcgen05" in build.sources()
                    and lib("attention_decode").kvad_attention_decode_takes_pre(self.code, int(head_dim), int(page_size)) == 1)

    def linear_sums(self, a, weight):
        """a . weight^T WITHOUT bias as 32-bit sums: the tensor-core product of a few rows splits K over CTAs, and where
        it has to store rounded results the CTAs of a split form a cluster and meet through shared memory; where it
        may ADD, they add their shares atomically and leave - half the time at GPT-2 XL's sizes.  So the product adds into one of two zeroed buffers, and the kernel that reads the sums (the
        decode attention: bias, rounding) clears the other one for the next such product (see `end_step`).  Returns (the sums [rows, outputs], the buffer to clear)."""
        m, n = a.shape[0], weight.shape[0]
        if self._sums is None or self._sums.shape[2] < n:
            if torch.cuda.is_current_stream_capturing():
                raise KernelError("linear_sums: its buffers must exist before a step is captured")
            self._sums = torch.zeros((2, 16, (n + 7) // 8 * 8), dtype=torch.float32, device=a.device)
        which = self._sum_calls % 2
        self._sum_calls += 1
        self._sums_open = True
        out = self._sums[which, :m, :n]
        self.linear(a, weight, None, out, "residual")
        return out, self._sums[1 - which]

    def attention_decode_sums(self, sums, bias, k_off: int, v_off: int, clear, out, row_seq, row_pos, page_table, k_pages,
                              v_pages, n_heads: int, scale: float, window: int = 0, *, n_splits: int = 1, scratch=None) -> None:
        """The decode attention with the rows' queries, keys and values given as `linear_sums` left them (queries from
        column 0, keys from `k_off`, values from `v_off`; `bias` as long as a row, or None): the kernel adds the bias,
        rounds, writes the rows' keys and values to the cache, merges its key ranges itself, and clears `clear`."""
        _need_cuda(sums, bias, clear, out, row_seq, row_pos, page_table, k_pages, v_pages, scratch)
        _, n_kv, page, hd = k_pages.shape
        n = sums.shape[0]
        ld_s, ld_o = _rows_view(sums, "q/k/v sums"), _rows_view(out, "attention output")
        if (sums.dtype != torch.float32 or out.dtype != self.dtype or k_pages.dtype != self.dtype or out.shape != (n, n_heads * hd)
                or k_off != n_heads * hd or v_off != k_off + n_kv * hd or sums.shape[1] != v_off + n_kv * hd):
            raise KernelError("attention_decode_sums: sums must be float32 [rows, q | k | v] and match heads x head size")
        bias_f32 = 0
        if bias is not None:
            if bias.numel() != sums.shape[1] or bias.dtype not in (torch.float32, torch.bfloat16):
                raise KernelError("attention_decode_sums: the bias must be as long as a row of sums, float32 or bfloat16")
            bias_f32 = 1 if bias.dtype == torch.float32 else 0
        if n_splits > 1 and (scratch is None or scratch.dtype != torch.float32 or scratch.numel() < n * n_heads * n_splits * (hd + 2)):
            raise KernelError("attention_decode_sums: scratch must be float32 with rows x heads x splits x (head_dim + 2) elements")
        counters = None
        if n_splits > 1:
            if self._counters is None or self._counters.numel() < n * n_heads:
                self._counters = torch.zeros(max(4096, n * n_heads), dtype=torch.int32, device=out.device)
            counters = self._counters
        h = lib("attention_decode")
        h.kvad_attention_decode_pre(_ptr(sums), ld_s, _ptr(bias), bias_f32, int(k_off), int(v_off), _ptr(clear),
                                    0 if clear is None else clear.numel())
        _check(h.kvad_attention_decode_step(self.code, c_void_p(0), 0, _ptr(out), ld_o, _ptr(row_seq), _ptr(row_pos),
                                            _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages),
                                            c_void_p(0), c_void_p(0), 0, _ptr(scratch), _ptr(counters), n, n_heads,
                                            n_kv, hd, page, int(n_splits), float(scale), int(window or 0), _stream()), h)

    # -- cache writes and attention --------------------------------------------------
    def kv_store(self, k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages) -> None:
        """Writes rows' keys and values to (sequence, position) in one layer's pages
        `[n_pages, n_kv_heads, page_size, head_dim]`."""
        _need_cuda(k_src, v_src, row_seq, row_pos, page_table, k_pages, v_pages)
        ld = _rows_view(k_src, "kv_store keys")
        if _rows_view(v_src, "kv_store values") != ld or k_src.shape != v_src.shape:
            raise KernelError("kv_store: keys and values must be views of one buffer with one row stride")
        _, n_kv, page, hd = k_pages.shape
        if k_src.shape[1] != n_kv * hd or k_pages.shape != v_pages.shape:
            raise KernelError("kv_store: rows do not match the cache's heads")
        if k_src.dtype != self.dtype or k_pages.dtype != self.dtype or not k_pages.is_contiguous() or not v_pages.is_contiguous():
            raise KernelError(f"kv_store: rows and pages must be {self.dtype}, pages contiguous")
        h = lib("rows")
        _check(h.kvad_kv_store(self.code, _ptr(k_src), _ptr(v_src), ld, _ptr(row_seq), _ptr(row_pos), _ptr(page_table),
                               page_table.shape[1], _ptr(k_pages), _ptr(v_pages), k_src.shape[0], n_kv, hd, page,
                               _stream()), h)

    def attention(self, q, out, row_seq, row_pos, page_table, k_pages, v_pages, n_heads: int, scale: float,
                  window: int = 0) -> None:
        """Every row attends over its own sequence's cached keys up to its own position
        (general kernel: any rows, any head size up to 512)."""
        _need_cuda(q, out, row_seq, row_pos, page_table, k_pages, v_pages)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or q.shape[0] != out.shape[0]:
            raise KernelError("attention: queries/output do not match heads x head size")
        if q.dtype != self.dtype or out.dtype != self.dtype or k_pages.dtype != self.dtype:
            raise KernelError(f"attention: tensors must be {self.dtype}")
        h = lib("attention_simt")
        _check(h.kvad_attention_simt(self.code, _ptr(q), ld_q, _ptr(out), ld_o, _ptr(row_seq), _ptr(row_pos),
                                     _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages), q.shape[0],
                                     n_heads, n_kv, hd, page, float(scale), int(window or 0), _stream()), h)

    def prompt_takes(self, head_dim: int, page_size: int) -> bool:
        """Whether the tiled CUDA-core kernel for prompts takes this head size and page size."""
        return head_dim % 4 == 0 and head_dim <= 256 and page_size == 64

    def attention_prompt(self, q, out, seq_starts, kv_lens, n_seqs: int, max_new: int, page_table, k_pages, v_pages,
                         n_heads: int, scale: float, window: int = 0) -> None:
        """Rows of sequences packed one after another (`seq_starts`), each sequence's rows being its last positions
        (`kv_lens` is its length after the step): causal attention on the CUDA cores in 32-bit arithmetic, a page of
        keys brought into shared memory once for 32 rows (the float32 engine's prompts; in bfloat16 the head sizes
        the tensor-core kernel refuses)."""
        _need_cuda(q, out, seq_starts, kv_lens, page_table, k_pages, v_pages)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or q.shape[0] != out.shape[0]:
            raise KernelError("attention_prompt: queries/output do not match heads x head size")
        if q.dtype != self.dtype or out.dtype != self.dtype or k_pages.dtype != self.dtype:
            raise KernelError(f"attention_prompt: tensors must be {self.dtype}")
        h = lib("attention_simt")
        _check(h.kvad_attention_tiled(self.code, _ptr(q), ld_q, _ptr(out), ld_o, _ptr(seq_starts), _ptr(kv_lens), _ptr(page_table),
                                      page_table.shape[1], _ptr(k_pages), _ptr(v_pages), int(n_seqs), n_heads, n_kv, hd, page,
                                      int(max_new), float(scale), int(window or 0), _stream()), h)

    PREFILL_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128)

    def prefill_takes(self, head_dim: int) -> bool:
        return head_dim in self.PREFILL_HEAD_SIZES

    def attention_prefill(self, q, out, seq_starts, kv_lens, n_seqs: int, max_new: int, page_table, k_pages, v_pages,
                          n_heads: int, scale: float, window: int = 0) -> None:
        """Rows of sequences packed one after another (`seq_starts`), each sequence's rows being its
        last positions (`kv_lens` is its length after the step): causal attention on the tensor cores."""
        _need_cuda(q, out, seq_starts, kv_lens, page_table, k_pages, v_pages)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or q.shape[0] != out.shape[0]:
            raise KernelError("attention_prefill: queries/output do not match heads x head size")
        if q.dtype != torch.bfloat16 or out.dtype != torch.bfloat16 or k_pages.dtype != torch.bfloat16:
            raise KernelError("attention_prefill: tensors must be bfloat16")
        h = lib("attention_prefill")
        _check(h.kvad_attention_prefill(_ptr(q), ld_q, q.shape[0], _ptr(out), ld_o, _ptr(seq_starts), _ptr(kv_lens),
                                        _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages),
                                        k_pages.shape[0], int(n_seqs), n_heads, n_kv, hd, page, int(max_new), float(scale),
                                        int(window or 0), _stream()), h)

    DECODE_HEAD_SIZES = (16, 32, 48, 64, 80, 96, 112, 128, 256)

    def decode_takes(self, head_dim: int) -> bool:
        return head_dim in self.DECODE_HEAD_SIZES

    @staticmethod
    def decode_splits(n_rows: int, n_heads: int, table_width: int, n_sms: Optional[int] = None) -> int:
        """Into how many key ranges a decode step cuts each (row, head): as many as keep the launch one wave
        of CTAs (2.75 an SM; three fit), six at most, one range per page at most.  Measured on a B200 at 12
        heads and ~520 keys, step time in ms by ranges: 4 rows 5: .308, 6: .311, 8: .322; 8 rows 4: .328,
        5: .353; 12 rows 2: .359, 3: .387; 16 rows 1: .394, 2: .366, 3: .405; 24 rows 1: .432, 2: .475.
        Depends on the batch's size only, never on lengths."""
        want = (11 * (n_sms or sm_count())) // (4 * max(1, n_rows * n_heads))
        return max(1, min(want, table_width, 6))          # (the splits of a row and head form one cluster: 8 at most)

    def attention_decode(self, q, out, row_seq, row_pos, page_table, k_pages, v_pages, n_heads: int, scale: float,
                         window: int = 0, *, n_splits: int = 1, scratch=None, k_new=None, v_new=None,
                         merge_in_kernel: bool = False) -> None:
        """Single-token rows over the cache, keys split over CTAs (decode kernel).

        `scratch`: float32, `n_rows * n_heads * n_splits * (head_dim + 2)` elements when `n_splits > 1`.
        `k_new` / `v_new`: this step's keys and values of the rows (views `[rows, kv_heads * head_dim]` of
        one buffer); given, the kernel reads each row's own position from them and writes it to the
        cache itself.  `merge_in_kernel`: the CTA that finishes last merges the splits (else a second kernel)."""
        _need_cuda(q, out, row_seq, row_pos, page_table, k_pages, v_pages, scratch, k_new, v_new)
        ld_q, ld_o = _rows_view(q, "attention queries"), _rows_view(out, "attention output")
        _, n_kv, page, hd = k_pages.shape
        n = q.shape[0]
        if q.shape[1] != n_heads * hd or out.shape[1] != n_heads * hd or out.shape[0] != n:
            raise KernelError("attention_decode: queries/output do not match heads x head size")
        if q.dtype != self.dtype or out.dtype != self.dtype or k_pages.dtype != self.dtype:
            raise KernelError(f"attention_decode: tensors must be {self.dtype}")
        if n_splits > 1 and (scratch is None or scratch.dtype != torch.float32
                             or scratch.numel() < n * n_heads * n_splits * (hd + 2)):
            raise KernelError("attention_decode: scratch must be float32 with rows x heads x splits x (head_dim + 2) elements")
        ld_new = 0
        if k_new is not None:
            ld_new = _rows_view(k_new, "new keys")
            if (v_new is None or _rows_view(v_new, "new values") != ld_new or k_new.shape != (n, n_kv * hd)
                    or v_new.shape != k_new.shape or k_new.dtype != self.dtype or v_new.dtype != self.dtype):
                raise KernelError("attention_decode: new keys and values must be views [rows, kv_heads x head size] of one buffer")
        counters = None
        if merge_in_kernel and n_splits > 1:
            if self._counters is None or self._counters.numel() < n * n_heads:
                self._counters = torch.zeros(max(4096, n * n_heads), dtype=torch.int32, device=q.device)
            counters = self._counters
        h = lib("attention_decode")
        _check(h.kvad_attention_decode_step(self.code, _ptr(q), ld_q, _ptr(out), ld_o, _ptr(row_seq), _ptr(row_pos),
                                            _ptr(page_table), page_table.shape[1], _ptr(k_pages), _ptr(v_pages),
                                            _ptr(k_new), _ptr(v_new), ld_new, _ptr(scratch), _ptr(counters), n, n_heads,
                                            n_kv, hd, page, int(n_splits), float(scale), int(window or 0), _stream()), h)
        if n_splits > 1 and counters is None:
            global _launches
            _launches += 1          # the merge kernel

    # -- sampling ------------------------------------------------------------------
    ARGMAX_CHUNK = 2048

    def argmax(self, logits, out, scratch=None) -> None:
        """out[r] = first index of the largest logit of row r.  With `scratch` (int64, rows x
        ceil(vocab / 2048) words) the rows are reduced by many blocks each, in two stages."""
        _need_cuda(logits, out, scratch)
        ld = _rows_view(logits, "argmax logits")
        n, vocab = logits.shape
        if logits.dtype != torch.float32 or out.dtype != torch.int32 or out.numel() < n:
            raise KernelError("argmax: logits must be float32 and the output int32, one per row")
        if scratch is not None and (scratch.dtype != torch.int64 or scratch.numel() < n * -(-vocab // self.ARGMAX_CHUNK)):
            raise KernelError("argmax: scratch must be int64 with rows x ceil(vocab / 2048) words")
        h = lib("sampling")
        _check(h.kvad_argmax(_ptr(logits), ld, n, vocab, _ptr(out), _ptr(scratch), _stream()), h)
        if scratch is not None:
            global _launches
            _launches += 1

    def sample(self, logits, temperature, top_k, top_p, uniform, out) -> None:
        """out[r] = token for row r: greedy where temperature[r] <= 0, else top-k, softmax at
        temperature, top-p, and the draw uniform[r] in [0, 1)."""
        _need_cuda(logits, temperature, top_k, top_p, uniform, out)
        ld = _rows_view(logits, "sample logits")
        n = logits.shape[0]
        ok = (logits.dtype == torch.float32 and temperature.dtype == torch.float32 and top_p.dtype == torch.float32
              and top_k.dtype == torch.int32 and uniform.dtype == torch.float32 and out.dtype == torch.int32
              and min(temperature.numel(), top_k.numel(), top_p.numel(), uniform.numel(), out.numel()) >= n)
        if not ok:
            raise KernelError("sample: needs float32 logits/temperature/top_p/uniform and int32 top_k/out, one per row")
        h = lib("sampling")
        _check(h.kvad_sample(_ptr(logits), ld, n, logits.shape[1], _ptr(temperature), _ptr(top_k), _ptr(top_p),
                             _ptr(uniform), _ptr(out), _stream()), h)


def sample_force_general(on: bool) -> None:
    """Tests: True sends every sampling row through the selections over the whole vocabulary, also
    where a small top-k has a shorter way."""
    switches_changed()
    h = lib("sampling")
    h.kvad_sample_force_general.argtypes = [c_int]
    h.kvad_sample_force_general.restype = None
    h.kvad_sample_force_general(int(bool(on)))


def prefill_force_legacy(on: bool) -> None:
    """Tests: True keeps the prompt attention of head sizes 64 and 128 on the mma.sync kernel, not the tcgen05 one."""
    switches_changed()
    h = lib("attention_prefill")
    h.kvad_attention_prefill_force_legacy.argtypes = [c_int]
    h.kvad_attention_prefill_force_legacy.restype = None
    h.kvad_attention_prefill_force_legacy(int(bool(on)))


def prefill_split_above(pages: int) -> None:
    """Tests and measurements: the tensor-core prompt attention gives a tile of 128 rows to both slots of a CTA,
    half of its pages each, when it sees more than `pages` pages (0: the kernel's own choice, 8)."""
    h = lib("attention_prefill")
    h.kvad_attention_prefill_split_above.argtypes = [c_int]
    h.kvad_attention_prefill_split_above.restype = None
    h.kvad_attention_prefill_split_above(int(pages))
    switches_changed()


def prefill_wait_timeouts() -> int:
    """How many bounded waits of the tcgen05 prompt attention have run out (0 in a healthy run)."""
    h = lib("attention_prefill")
    h.kvad_attention_prefill_status.argtypes = []
    h.kvad_attention_prefill_status.restype = c_int
    n = h.kvad_attention_prefill_status()
    if n < 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))
    return n


def decode_force_plain(on) -> None:
    """Tests: 1 / True keeps the decode attention of every head size on the kernel that loads through
    registers; 2 keeps the TMA-fed kernel but merges splits through global memory, not a cluster; 0: default."""
    switches_changed()
    h = lib("attention_decode")
    h.kvad_attention_decode_force_plain.argtypes = [c_int]
    h.kvad_attention_decode_force_plain.restype = None
    h.kvad_attention_decode_force_plain(int(on))


def decode_wait_timeouts() -> int:
    """How many bounded waits of the TMA-fed decode attention have run out (0 in a healthy run)."""
    h = lib("attention_decode")
    h.kvad_attention_decode_status.argtypes = []
    h.kvad_attention_decode_status.restype = c_int
    n = h.kvad_attention_decode_status()
    if n < 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))
    return n


def tcgen05_load_form(mode: int) -> None:
    """Tests: 0 lets the swapped linear kernel choose between one TMA load per K block and grouped
    three-dimensional loads; 1 forces the former, 2 the latter (where K is a multiple of 64)."""
    switches_changed()
    h = lib("linear_tcgen05")
    h.kvad_linear_tcgen05_no_3d.argtypes = [c_int]
    h.kvad_linear_tcgen05_no_3d.restype = None
    h.kvad_linear_tcgen05_no_3d(int(mode))


def tcgen05_cluster_k(on: bool) -> None:
    """Tests: False keeps K whole under the storing epilogues of the swapped form (no reduction inside a cluster)."""
    switches_changed()
    h = build.load("linear_tcgen05")
    h.kvad_linear_tcgen05_no_cluster_k.argtypes = [c_int]
    h.kvad_linear_tcgen05_no_cluster_k.restype = None
    h.kvad_linear_tcgen05_no_cluster_k(int(not on))


def tcgen05_plain_stores(on: bool) -> None:
    """Tests: the wide linear kernel writes its output with plain stores instead of TMA stores / reduce-adds."""
    switches_changed()
    h = lib("linear_tcgen05")
    h.kvad_linear_tcgen05_no_tma_out.argtypes = [c_int]
    h.kvad_linear_tcgen05_no_tma_out.restype = None
    h.kvad_linear_tcgen05_no_tma_out(int(bool(on)))


def tcgen05_test_hooks(wait_limit: int = 0, skip_first_load: bool = False) -> None:
    """Tests of the bounded waits of the tensor-core linear kernel: `wait_limit` polls before a wait gives up
    (0: the library's own limit); `skip_first_load`: the next launch of the swapped form (17..64 rows) leaves
    out its first load, so its wait for it runs out and the launch returns with the status counter raised."""
    h = lib("linear_tcgen05")
    h.kvad_linear_tcgen05_test_hooks.argtypes = [ctypes.c_uint, c_int]
    h.kvad_linear_tcgen05_test_hooks.restype = c_int
    if h.kvad_linear_tcgen05_test_hooks(int(wait_limit), int(bool(skip_first_load))) != 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))


def tcgen05_wait_timeouts() -> int:
    """How many bounded waits of the tensor-core linear kernel have run out (0 in a healthy run)."""
    h = lib("linear_tcgen05")
    n = h.kvad_linear_tcgen05_status()
    if n < 0:
        raise KernelError(h.kvad_last_error().decode("utf-8", "replace"))
    return n


def tcgen05_takes(a, weight, out, lda: int, ldo: int) -> bool:
    """Shapes the tensor-core linear kernel accepts: TMA wants 16-byte aligned
    bases and row strides (bfloat16: multiples of 8 elements)."""
    k = a.shape[1]
    return (k % 8 == 0 and lda % 8 == 0 and a.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and out.data_ptr() % 16 == 0)
