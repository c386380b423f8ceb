"""Python face of the CUDA kernel library: one function per C entry point.

Arguments are torch tensors on a CUDA device; each function checks device,
dtype and layout, passes raw pointers and the current stream, and raises
:class:`KernelError` with the library's message when a kernel refuses its
sizes.  Nothing here computes on the host and nothing falls back to torch.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc import KernelLibraryError, load_library
from .kernels_const import PAGE

F32, BF16 = 0, 1
ACTIVATIONS = {"gelu_tanh": 0, "silu": 1}
PAIRINGS = {"half": 0, "adjacent": 1}


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _lib():
    return load_library()


def _stream() -> c_void_p:
    # the raw handle of the current stream of the current device (the Stream object of
    # torch.cuda.current_stream() costs several microseconds a call, once per kernel launched)
    return c_void_p(_raw_stream(_current_device()))


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)
if _raw_stream is None or _current_device is None:          # an older or newer torch: the documented way
    def _raw_stream(_index):                                 # noqa: F811
        return torch.cuda.current_stream().cuda_stream

    def _current_device():                                   # noqa: F811
        return 0


def _ptr(t, name="tensor", dtype=None, allow_none=False) -> c_void_p:
    if t is None:
        if allow_none:
            return c_void_p(0)
        raise KernelError(f"{name} is required")
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU implementation)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    return c_void_p(t.data_ptr())


def _rows(t, name) -> int:
    """Row stride in elements of a 2-D tensor whose rows are dense."""
    if t.dim() != 2 or t.stride(1) != 1:
        raise KernelError(f"{name} must be 2-D with dense rows, got shape {tuple(t.shape)} strides {t.stride()}")
    return t.stride(0)


def _check(code: int) -> None:
    if code != 0:
        msg = _lib().af_last_error().decode("utf-8", "replace")
        raise KernelError(f"{msg} (code {code})")


def launch_count() -> int:
    """Kernels this library has launched since it was loaded."""
    f = _lib().af_launch_count
    f.restype = ctypes.c_ulonglong
    return int(f())


def bounds_failures():
    """The checked build's record (see ``csrc.use_checked_build``): None in the
    normal build, else (translation units that saw a bad index since the last
    call, one of the bad values).  Synchronises the device."""
    index = c_int(0)
    n = int(_lib().af_bounds_failures(ctypes.byref(index)))
    if n < 0:
        return None
    return n, int(index.value)


_SMS = {}


def sm_count() -> int:
    """Streaming multiprocessors of the current device (asked of the driver
    once per device): what the policies that cut work into blocks divide by."""
    dev = _current_device()
    n = _SMS.get(dev)
    if n is None:
        n = int(_lib().af_device_sm_count())
        if n <= 0:
            _check(n or -1)
        _SMS[dev] = n
    return n


def require_cuda_tensor(t, name="tensor"):
    if not t.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device")


# ---------------------------------------------------------------- elementwise

def embed(out, table, ids, scale: float) -> None:
    """out[t] = table[ids[t]] * scale; out float32 [T, H]."""
    T, H = out.shape
    _check(_lib().af_embed(_ptr(out, "out", torch.float32), _ptr(table, "table"), c_int(dtype_code(table.dtype)),
                           _ptr(ids, "ids", torch.int32), c_int(T), c_int(H), c_int(table.shape[0]),
                           c_float(scale), _stream()))


def rmsnorm(y, x, w, eps: float, offset: float, rows=None) -> None:
    """y[r] = norm(x[rows[r]] or x[r]) * (offset + w); x, w float32."""
    n, H = y.shape
    if not (x.is_contiguous() and y.is_contiguous()):
        raise KernelError("rmsnorm: tensors must be contiguous")
    _check(_lib().af_rmsnorm(_ptr(y, "y"), c_int(dtype_code(y.dtype)), _ptr(x, "x", torch.float32),
                             _ptr(w, "w", torch.float32), _ptr(rows, "rows", torch.int32, allow_none=True),
                             c_int(n), c_int(H), c_float(eps), c_float(offset), _stream()))


def add_rmsnorm(x, a, w_post, eps_post: float, offset: float, y=None, w_next=None, eps_next: float = 0.0,
                n_parts: int = 1) -> None:
    """x += norm(a) * (offset + w_post); if y: y = norm(x) * (offset + w_next).
    With ``n_parts`` > 1, ``a`` is float32 [n_parts, rows, H] partial sums."""
    n, H = x.shape
    if not (x.is_contiguous() and a.is_contiguous() and (y is None or y.is_contiguous())):
        raise KernelError("add_rmsnorm: tensors must be contiguous")
    part_stride = n * H
    _check(_lib().af_add_rmsnorm(_ptr(x, "x", torch.float32), _ptr(a, "a"), c_int(dtype_code(a.dtype)),
                                 c_int(n_parts), c_longlong(part_stride), _ptr(w_post, "w_post", torch.float32),
                                 _ptr(y, "y", allow_none=True), c_int(dtype_code(y.dtype) if y is not None else F32),
                                 _ptr(w_next, "w_next", torch.float32, allow_none=True),
                                 c_int(n), c_int(H), c_float(eps_post), c_float(eps_next), c_float(offset),
                                 _stream()))


def gated_act(out, gu, activation: str) -> None:
    """out[m, i] = act(gu[m, i]) * gu[m, I + i]."""
    n, inter = out.shape
    if gu.shape != (n, 2 * inter) or not (gu.is_contiguous() and out.is_contiguous()) or gu.dtype != out.dtype:
        raise KernelError("gated_act: gu must be contiguous [rows, 2 * inter] of out's dtype")
    if activation not in ACTIVATIONS:
        raise KernelError(f"gated_act: unknown activation '{activation}' (known: {sorted(ACTIVATIONS)})")
    _check(_lib().af_gated_act(_ptr(out), _ptr(gu), c_int(dtype_code(out.dtype)), c_int(n), c_int(inter),
                               c_int(ACTIVATIONS[activation]), _stream()))


def softcap_(z, cap: float) -> None:
    if not z.is_contiguous():
        raise KernelError("softcap_: tensor must be contiguous")
    _check(_lib().af_softcap(_ptr(z, "z", torch.float32), c_longlong(z.numel()), c_float(cap), _stream()))


# ---------------------------------------------------------------- matrix product

def gemm_plain(out, x, w, cap: float = 0.0) -> None:
    """out[M, N] = x[M, K] @ w[N, K]^T on the CUDA cores, 32-bit accumulation;
    x and w share a dtype, out is that dtype or float32."""
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or out.shape != (M, N) or x.dtype != w.dtype:
        raise KernelError(f"gemm_plain: shapes {tuple(x.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _check(_lib().af_gemm_plain(_ptr(out), c_int(dtype_code(out.dtype)), c_int(_rows(out, "out")),
                                _ptr(x), c_int(_rows(x, "x")), _ptr(w), c_int(_rows(w, "w")),
                                c_int(dtype_code(x.dtype)), c_int(M), c_int(N), c_int(K), c_float(cap),
                                _stream()))


# ---------------------------------------------------------------- attention

ROPE_TABLE_ROWS = 64     # from this many rows on, the rotary kernel for bfloat16 rows takes the step's table


def rope_cache_write(qkv, positions, inv_freq, nq: int, nkv: int, hd: int, rot_dim: int, pairing: str,
                     seq_of_token=None, slots=None, len_after=None, kcache=None, vcache=None,
                     page_table=None, ring_rows: int = 0, parts=None, table=None) -> None:
    """Rotate the q and k heads of the packed rows [q | k | v] in place and,
    when a cache is given, store k and v at each token's row of its page.
    ``parts`` (float32 [S, T, width] split-K partial sums) are added into qkv first.
    ``table``: the step's cosines and sines (:func:`rope_table` of these positions and
    frequencies); the kernel for many bfloat16 rows reads them instead of working them
    out for every layer again (the same 32-bit values)."""
    T = qkv.shape[0]
    if qkv.shape[1] != (nq + 2 * nkv) * hd:
        raise KernelError(f"rope_cache_write: row width {qkv.shape[1]} is not (nq + 2 nkv) * head_dim")
    if pairing not in PAIRINGS:
        raise KernelError(f"rope_cache_write: unknown pairing '{pairing}'")
    if inv_freq.numel() != rot_dim // 2:
        raise KernelError("rope_cache_write: inv_freq must hold rot_dim / 2 values")
    if table is not None and (tuple(table.shape) != (T, rot_dim // 2, 2) or not table.is_contiguous()):
        raise KernelError(f"rope_cache_write: the table must be [{T}, {rot_dim // 2}, 2]")
    max_pages = 0
    if kcache is not None:
        if kcache.dtype != qkv.dtype or vcache.dtype != qkv.dtype:
            raise KernelError("rope_cache_write: cache dtype differs from the activations'")
        if tuple(kcache.shape[1:]) != (nkv, PAGE, hd) or not kcache.is_contiguous() or not vcache.is_contiguous():
            raise KernelError(f"rope_cache_write: cache pages must be [pages, {nkv}, {PAGE}, {hd}]")
        max_pages = page_table.shape[1]
    _check(_lib().af_rope_cache_write(
        _ptr(qkv), c_int(dtype_code(qkv.dtype)), c_int(_rows(qkv, "qkv")),
        _ptr(parts, "parts", torch.float32, allow_none=True), c_int(parts.shape[0] if parts is not None else 0),
        c_longlong(parts.stride(0) if parts is not None else 0), _ptr(positions, "positions", torch.int32),
        _ptr(seq_of_token, "seq_of_token", torch.int32, allow_none=True),
        _ptr(slots, "slots", torch.int32, allow_none=True),
        _ptr(len_after, "len_after", torch.int32, allow_none=True),
        _ptr(inv_freq, "inv_freq", torch.float32), _ptr(table, "table", torch.float32, allow_none=True),
        c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_int(rot_dim),
        c_int(PAIRINGS[pairing]), _ptr(kcache, allow_none=True), _ptr(vcache, allow_none=True),
        _ptr(page_table, "page_table", torch.int32, allow_none=True), c_int(max_pages), c_int(ring_rows),
        _stream()))


_EMPTY_F32 = {}


def _no_frequencies(device):
    key = str(device)
    if key not in _EMPTY_F32:
        _EMPTY_F32[key] = torch.empty(0, dtype=torch.float32, device=device)
    return _EMPTY_F32[key]


def store_kv(qkv, batch, nq: int, nkv: int, hd: int, kv, parts=None) -> None:
    """A mixer's cache store: the k and v heads of the packed rows [q | k | v]
    go to each token's row of its cache page (``kv``: the layer's view of its
    pages).  ``parts`` (split-K partial sums of the rows) are added into
    ``qkv`` first.  Nothing is rotated."""
    rope_cache_write(qkv, batch.positions, _no_frequencies(qkv.device), nq, nkv, hd, 0, "half",
                     seq_of_token=batch.seq_of_token, slots=batch.slots, len_after=batch.len_after,
                     kcache=kv.k, vcache=kv.v, page_table=kv.page_table, ring_rows=kv.ring_rows, parts=parts)


def sum_parts(qkv, parts, batch, nq: int, nkv: int, hd: int) -> None:
    """qkv = the sum of the split-K partial sums ``parts`` (float32 [S, T, width]), in index order."""
    rope_cache_write(qkv, batch.positions, _no_frequencies(qkv.device), nq, nkv, hd, 0, "half", parts=parts)


def attn_prefill_plain(out, q, k, v, positions, nq: int, nkv: int, hd: int, scale: float, cap: float,
                       window: int, slopes=None) -> None:
    """Attention of prompts that start at position 0 over the step's own keys.
    q [T, nq*hd], k/v [T, nkv*hd] are row views (any row stride).  ``slopes``
    (float32 [nq]): slope[h] * (key position - query position) is added to head
    h's scores after scale and cap (a position encoding that biases scores)."""
    if slopes is not None and slopes.numel() != nq:
        raise KernelError(f"attn_prefill_plain: {slopes.numel()} slopes for {nq} heads")
    T = q.shape[0]
    _check(_lib().af_attn_prefill_plain(
        _ptr(out), c_int(_rows(out, "out")), _ptr(q), c_int(_rows(q, "q")), _ptr(k), c_int(_rows(k, "k")),
        _ptr(v), c_int(_rows(v, "v")), c_int(dtype_code(q.dtype)), _ptr(positions, "positions", torch.int32),
        c_int(T), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_float(cap), c_int(window),
        _ptr(slopes, "slopes", torch.float32, allow_none=True), _stream()))


def attn_decode_plain(out, q, kcache, vcache, page_table, slots, lens, nq: int, nkv: int, hd: int,
                      scale: float, cap: float, window: int, ring_rows: int, slopes=None) -> None:
    """Attention of one new token per sequence over the cache pages
    (``slopes`` as in :func:`attn_prefill_plain`)."""
    B = q.shape[0]
    if slopes is not None and slopes.numel() != nq:
        raise KernelError(f"attn_decode_plain: {slopes.numel()} slopes for {nq} heads")
    if kcache.dtype != q.dtype:
        raise KernelError("attn_decode_plain: cache dtype differs from the activations'")
    _check(_lib().af_attn_decode_plain(
        _ptr(out), c_int(_rows(out, "out")), _ptr(q), c_int(_rows(q, "q")), _ptr(kcache), _ptr(vcache),
        c_int(dtype_code(q.dtype)), _ptr(page_table, "page_table", torch.int32), c_int(page_table.shape[1]),
        _ptr(slots, "slots", torch.int32), _ptr(lens, "lens", torch.int32), c_int(B), c_int(nq), c_int(nkv),
        c_int(hd), c_float(scale), c_float(cap), c_int(window), c_int(ring_rows),
        _ptr(slopes, "slopes", torch.float32, allow_none=True), _stream()))


def add_(x, a) -> None:
    """x += a; x float32, a float32 or bfloat16, same shape (or [S, *x.shape]
    partial sums, added one after the other)."""
    if a.dim() == x.dim() + 1:
        for part in a:
            add_(x, part)
        return
    if x.shape != a.shape or not (x.is_contiguous() and a.is_contiguous()):
        raise KernelError("add_: tensors must be contiguous and of one shape")
    _check(_lib().af_add(_ptr(x, "x", torch.float32), _ptr(a), c_int(dtype_code(a.dtype)),
                         c_longlong(x.numel()), _stream()))


def sample(logits, out, temperature: float, top_p: float, penalty: float, uniform=None, recent=None,
           n_recent=None) -> None:
    """One token per row of float32 logits [R, V] into out int32 [R].  The
    repetition penalty changes ``logits`` in place.  ``recent`` int32 [R, 64]
    holds each row's last tokens, ``n_recent`` int32 [R] how many are valid,
    ``uniform`` float32 [R] the draws in [0, 1)."""
    R, V = logits.shape
    if out.shape[0] != R:
        raise KernelError("sample: one output per row")
    _check(_lib().af_sample(_ptr(logits, "logits", torch.float32), c_int(_rows(logits, "logits")), c_int(R),
                            c_int(V), _ptr(recent, "recent", torch.int32, allow_none=True),
                            _ptr(n_recent, "n_recent", torch.int32, allow_none=True),
                            c_int(recent.stride(0) if recent is not None else 0), c_float(temperature),
                            c_float(top_p), c_float(penalty),
                            _ptr(uniform, "uniform", torch.float32, allow_none=True),
                            _ptr(out, "out", torch.int32), _stream()))


_ERR = {}


def error_word(device) -> torch.Tensor:
    """The device word that kernels set when a bounded wait inside them ran out."""
    key = torch.device(device).index or 0
    if key not in _ERR:
        _ERR[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _ERR[key]


def check_device_errors(device) -> None:
    """Raise if a kernel reported a wait that ran out of time (reads one word: synchronises)."""
    w = error_word(device)
    if int(w.item()) != 0:
        w.zero_()
        raise KernelError("a tensor-core kernel gave up waiting on a barrier (results of the step are invalid)")


def selftest_wait_runs_out(device, limit_ms: float = 2.0) -> float:
    """Runs a kernel whose wait on a barrier nobody arrives on gives up after
    ``limit_ms`` and sets the device's error word, as the tensor-core kernels'
    waits do after their limit.  Returns the milliseconds the wait took; the
    error word is left set (``check_device_errors`` raises and clears it)."""
    waited = torch.zeros(1, dtype=torch.int64, device=device)
    _check(_lib().af_selftest_wait_runs_out(_ptr(error_word(device), "err", torch.int32),
                                            ctypes.c_ulonglong(int(limit_ms * 1e6)), _ptr(waited), _stream()))
    return float(waited.item()) / 1e6


def gemm_tc_supported(x, w, out) -> bool:
    """Whether the tensor-core product takes these operands: bfloat16, dense
    rows, K and row strides multiples of 8, 16-byte aligned bases."""
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if x.dim() != 2 or w.dim() != 2 or x.stride(1) != 1 or w.stride(1) != 1:
        return False
    K = x.shape[1]
    return (K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0 and (out is None or out.stride(-1) == 1))


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """How many K splits fill the GPU when a product has few output tiles: up to
    two blocks an SM (a grid beyond one wave runs two blocks an SM, which stream
    at once: measured faster inside the decode step than one wave of blocks
    with a whole SM each; for up to 16 rows), at least 4 K blocks a split, at
    most 16 splits."""
    lib = _lib()
    bn = lib.af_gemm_tc_token_tile(c_int(M))
    tiles = ((N + 127) // 128) * ((M + bn - 1) // bn)
    kb = (K + 63) // 64
    if tiles >= 96 or kb < 8:
        return 1
    waves = 2 if M <= 16 else 1       # (more rows: the partial sums' own bytes weigh more than the fuller GPU)
    want = max(1, min((waves * sm_count()) // tiles, kb // 4, 16))
    per = (kb + want - 1) // want
    return (kb + per - 1) // per


# Blocks per SM of the weight-bound product (up to 64 tokens): 0 lets the library choose.
GEMM_TC_PER_SM = 0


def gemm_tc(out, x, w, cap: float = 0.0, splits: int = 1, gated: bool = False, activation: str = "gelu_tanh",
            n_acc: int = 0, checked: bool = False, per_sm: int = -1) -> None:
    """out = x @ w^T on the tcgen05 tensor cores (bfloat16 operands, 32-bit
    accumulation in TMEM).  splits > 1: out is float32 [splits, M, N] partial
    sums.  gated: w holds, per group of 32 rows, 16 gate rows then the 16 up
    rows of the same features (see ``interleave_gate_up``); out[m, f] =
    act(x . gate_f) * (x . up_f), N = rows / 2.  n_acc: weight tiles per block
    (1 or 2), or 4: the kernel that runs a tile on a pair of SMs
    (``tcgen05.mma.cta_group::2``, two accumulators in turn: for prompts);
    0: chosen from the sizes.  ``checked``: the caller has asked
    :func:`gemm_tc_supported` already."""
    M, K = x.shape
    rows = w.shape[0]
    N = rows // 2 if gated else rows
    if not checked and not gemm_tc_supported(x, w, out):
        raise KernelError("gemm_tc: operands must be bfloat16 with dense, 16-byte aligned rows and K % 8 == 0")
    if splits > 1:
        if out.dtype != torch.float32 or tuple(out.shape) != (splits, M, N) or not out.is_contiguous():
            raise KernelError("gemm_tc: split-K wants a contiguous float32 [splits, M, N] output")
        ldo, part = N, M * N
    else:
        if tuple(out.shape) != (M, N):
            raise KernelError(f"gemm_tc: output shape {tuple(out.shape)}, expected {(M, N)}")
        ldo, part = out.stride(0), 0
    if n_acc == 0:
        # Many tokens.  Two weight tiles per block halve the bytes a block stages per flop; worth it once the
        # tiles of 256 x 256 fill the GPU.  With fewer tiles and a long K a tile runs on a pair of SMs (the same
        # bytes per flop, 128 rows a block); with a short K the pair's set-up costs what it saves.  Measured at
        # 2,048 tokens on a B200: 18432 x 2304 gated 122 us / 124 us / 132 us (two tiles / pair / one tile),
        # 2304 x 9216 90 / 59 / 63, 2304 x 2048 25 / 17 / 15, 4096 x 2304 31 / 31 / 31.
        blocks2 = ((rows + 255) // 256) * ((M + 255) // 256)
        n_acc = 1
        if M > 128 and splits == 1:
            if blocks2 >= 120:
                n_acc = 2
            elif blocks2 >= 60 and K >= 4096:
                n_acc = 4
    if n_acc == 4:
        if splits > 1:
            raise KernelError("gemm_tc: the kernel on pairs of SMs does not split K")
        _check(_lib().af_gemm_tc_pair(_ptr(out), c_int(dtype_code(out.dtype)), c_longlong(ldo), _ptr(x),
                                      c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)), c_longlong(rows),
                                      c_int(M), c_int(K), c_int(1 if gated else 0), c_int(ACTIVATIONS[activation]),
                                      c_float(cap), _ptr(error_word(x.device), "err", torch.int32), _stream()))
        return
    _check(_lib().af_gemm_tc(_ptr(out), c_int(dtype_code(out.dtype)), c_longlong(ldo), c_longlong(part), _ptr(x),
                             c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)), c_longlong(rows),
                             c_int(M), c_int(K), c_int(1 if gated else 0), c_int(ACTIVATIONS[activation]),
                             c_int(n_acc), c_float(cap), c_int(splits), c_int(GEMM_TC_PER_SM if per_sm < 0 else per_sm),
                             _ptr(error_word(x.device), "err", torch.int32), _stream()))


def rope_table(positions, inv_freq) -> torch.Tensor:
    """float32 [T, pairs, 2]: (cos, sin) of position * frequency for every token
    of the step and every rotary pair (32-bit angles)."""
    T, half = positions.shape[0], inv_freq.numel()
    table = torch.empty(T, half, 2, dtype=torch.float32, device=positions.device)
    _check(_lib().af_rope_table(_ptr(table), _ptr(positions, "positions", torch.int32),
                                _ptr(inv_freq, "inv_freq", torch.float32), c_int(T), c_int(half), _stream()))
    return table


def kv_rows(batch, kv, nkv: int) -> torch.Tensor:
    """int32 [T]: each token's row in the cache pages of ``kv`` (a layer's view;
    all layers of its group share the page table) for kv head 0, -1 for tokens
    that are not stored."""
    T = batch.tokens.shape[0]
    rows = torch.empty(T, dtype=torch.int32, device=batch.tokens.device)
    _check(_lib().af_kv_rows(_ptr(rows), _ptr(batch.positions, "positions", torch.int32),
                             _ptr(batch.seq_of_token, "seq_of_token", torch.int32),
                             _ptr(batch.slots, "slots", torch.int32), _ptr(batch.len_after, "len_after", torch.int32),
                             _ptr(kv.page_table, "page_table", torch.int32), c_int(kv.page_table.shape[1]),
                             c_int(kv.ring_rows), c_int(nkv), c_int(T), _stream()))
    return rows


def rope_row_order(n_heads: int, hd: int, device=None) -> torch.Tensor:
    """The order of a packed [q | k | v] weight's rows that :func:`gemm_tc_rope`
    wants: within every head, groups of 32 rows, each the 16 rows p .. p + 15
    of the head's first half followed by the rows p + hd / 2 .. that they are
    rotated with.  Returns the old row index of every new row (int64)."""
    if hd % 32:
        raise KernelError(f"rope_row_order: head_dim {hd} is not a multiple of 32")
    i = torch.arange(hd, device=device)
    within = (i // 32) * 16 + i % 16 + (i % 32 >= 16) * (hd // 2)
    return (torch.arange(n_heads, device=device)[:, None] * hd + within[None, :]).reshape(-1)


def gemm_tc_rope_supported(x, w, hd: int) -> bool:
    return hd % 32 == 0 and gemm_tc_supported(x, w, None)


def gemm_tc_rope(out, x, w, table, nq: int, nkv: int, hd: int, rows=None, kcache=None, vcache=None,
                 splits: int = 1, tickets=None, n_acc: int = 0, per_sm: int = -1) -> None:
    """out [M, (nq + 2 nkv) hd] bfloat16 = x @ w^T with the rotary encoding and
    the cache write in the product's epilogue: ``w`` holds the rows in
    :func:`rope_row_order`, ``table`` is :func:`rope_table` of the step; q and k
    heads are rotated (pairs i, i + hd / 2), v is not; ``out`` is in the plain
    order.  With ``rows`` (:func:`kv_rows`) and the layer's cache pages, k and v
    also go to each token's cache row.  ``splits`` > 1 (up to 64 tokens): the
    last block of a tile to finish adds the partial tiles in index order;
    ``tickets`` is a zeroed int32 tensor that the kernel leaves zeroed."""
    M, K = x.shape
    N = w.shape[0]
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N) or N != (nq + 2 * nkv) * hd:
        raise KernelError(f"gemm_tc_rope: output {tuple(out.shape)} for {(M, (nq + 2 * nkv) * hd)}")
    if not gemm_tc_rope_supported(x, w, hd):
        raise KernelError("gemm_tc_rope: operands must be bfloat16 with dense, 16-byte aligned rows, K % 8 == 0 "
                          "and head_dim % 32 == 0")
    if tuple(table.shape) != (M, hd // 2, 2) or table.dtype != torch.float32 or not table.is_contiguous():
        raise KernelError(f"gemm_tc_rope: the table must be float32 [{M}, {hd // 2}, 2]")
    if rows is not None:
        if kcache is None or vcache is None or kcache.dtype != torch.bfloat16 or not kcache.is_contiguous() \
                or tuple(kcache.shape[1:]) != (nkv, PAGE, hd) or vcache.shape != kcache.shape:
            raise KernelError(f"gemm_tc_rope: cache pages must be bfloat16 [pages, {nkv}, {PAGE}, {hd}]")
    parts = None
    if splits > 1:
        need = int(_lib().af_gemm_tc_rope_tickets(c_int(M), c_longlong(N)))
        if M > 64 or tickets is None or tickets.dtype != torch.int32 or tickets.numel() < need:
            raise KernelError(f"gemm_tc_rope: split-K serves up to 64 tokens and needs {need} zeroed int32 tickets")
        parts = torch.empty(splits, M, N, dtype=torch.float32, device=x.device)
    if n_acc == 0:
        blocks2 = ((N + 255) // 256) * ((M + 255) // 256)
        n_acc = 2 if (M > 128 and splits == 1 and blocks2 >= 120) else 1
    _check(_lib().af_gemm_tc_rope(
        _ptr(out), c_longlong(out.stride(0)), _ptr(x), c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)),
        c_longlong(N), c_int(M), c_int(K), c_int(n_acc), c_int(splits),
        _ptr(parts, "parts", torch.float32, allow_none=True), _ptr(tickets, "tickets", torch.int32, allow_none=True),
        _ptr(table, "table", torch.float32), _ptr(rows, "rows", torch.int32, allow_none=True),
        _ptr(kcache, allow_none=True), _ptr(vcache, allow_none=True), c_int(hd), c_int(nq), c_int(nkv),
        c_int(GEMM_TC_PER_SM if per_sm < 0 else per_sm), _ptr(error_word(x.device), "err", torch.int32), _stream()))


def argmax_key_stride() -> int:
    """64-bit words between the keys of two rows of :func:`gemm_tc_argmax`."""
    return int(_lib().af_argmax_key_stride())


def gemm_tc_argmax(tokens, x, w, cap: float, keys) -> None:
    """tokens[m] = argmax over the rows n of softcap(x[m] . w[n]) (finite values
    only, the lowest row among equals, 0 when none is finite), without the
    logits going to memory: the product's epilogue joins every block's best
    into one 64-bit key per token.  ``keys``: int64 [>= M] on the device, zero
    before the call and zero again after it."""
    M, K = x.shape
    if not gemm_tc_supported(x, w, None):
        raise KernelError("gemm_tc_argmax: operands must be bfloat16 with dense, 16-byte aligned rows and K % 8 == 0")
    if tokens.dtype != torch.int32 or tokens.numel() < M or keys.dtype != torch.int64 \
            or keys.numel() < M * argmax_key_stride():
        raise KernelError("gemm_tc_argmax: int32 tokens, one per row, and int64 keys, argmax_key_stride() per row")
    lib = _lib()
    _check(lib.af_gemm_tc_argmax(_ptr(keys), _ptr(x), c_longlong(x.stride(0)), _ptr(w), c_longlong(w.stride(0)),
                                 c_longlong(w.shape[0]), c_int(M), c_int(K), c_float(cap), c_int(max(GEMM_TC_PER_SM, 0)),
                                 _ptr(error_word(x.device), "err", torch.int32), _stream()))
    _check(lib.af_argmax_finish(_ptr(tokens), _ptr(keys), c_int(M), _stream()))


def interleave_gate_up(w_gate, w_up):
    """The gated product's weight layout: groups of 32 rows, each 16 gate rows
    followed by the up rows of the same 16 features.  Rows beyond the last
    whole 16 are padded with zeros (their outputs are never written)."""
    inter, K = w_gate.shape
    groups = (inter + 15) // 16
    out = torch.zeros(groups * 32, K, dtype=w_gate.dtype, device=w_gate.device)
    v = out.view(groups, 2, 16, K)
    pad = groups * 16 - inter
    if pad:
        g = torch.cat([w_gate, torch.zeros(pad, K, dtype=w_gate.dtype, device=w_gate.device)])
        u = torch.cat([w_up, torch.zeros(pad, K, dtype=w_up.dtype, device=w_up.device)])
    else:
        g, u = w_gate, w_up
    v[:, 0] = g.view(groups, 16, K)
    v[:, 1] = u.view(groups, 16, K)
    return out

def attn_prefill_mma(out, q, k, v, seq_starts, n_seqs: int, max_len: int, nq, nkv, hd, scale, cap, window) -> None:
    """bfloat16 prefill attention on the tensor cores; sequences packed row
    after row, ``seq_starts`` int32 [n_seqs + 1]."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_mma: bfloat16 only")
    _check(_lib().af_attn_prefill(
        _ptr(out), c_longlong(_rows(out, "out")), _ptr(q), c_longlong(_rows(q, "q")), _ptr(k),
        c_longlong(_rows(k, "k")), _ptr(v), c_longlong(_rows(v, "v")), _ptr(seq_starts, "seq_starts", torch.int32),
        c_int(n_seqs), c_int(max_len), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_float(cap), c_int(window),
        _stream()))


def attn_prefill_tc(out, q, k, v, seq_starts, n_seqs: int, max_len: int, nq, nkv, hd, scale, cap, window) -> None:
    """bfloat16 prefill attention on tcgen05 (S and O in TMEM); sequences packed
    row after row, ``seq_starts`` int32 [n_seqs + 1]."""
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_prefill_tc: bfloat16 only")
    if k.shape[0] != q.shape[0] or v.shape[0] != q.shape[0]:
        raise KernelError("attn_prefill_tc: q, k and v hold the same rows")
    _check(_lib().af_attn_prefill_tc(
        _ptr(out), c_longlong(_rows(out, "out")), _ptr(q), c_longlong(_rows(q, "q")), _ptr(k),
        c_longlong(_rows(k, "k")), _ptr(v), c_longlong(_rows(v, "v")), _ptr(seq_starts, "seq_starts", torch.int32),
        c_int(n_seqs), c_int(q.shape[0]), c_int(max_len), c_int(nq), c_int(nkv), c_int(hd), c_float(scale),
        c_float(cap), c_int(window), _ptr(error_word(q.device), "err", torch.int32), _stream()))


def attn_prefill(out, q, k, v, batch, nq, nkv, hd, scale, cap, window, slopes=None) -> None:
    """Attention of a prefill step: for bfloat16 the tcgen05 kernel (head sizes
    128, 256) or the mma.sync kernel (64), else the plain kernel (which also
    serves scores with a per-head slope)."""
    if slopes is not None:
        attn_prefill_plain(out, q, k, v, batch.positions, nq, nkv, hd, scale, cap, window, slopes)
        return
    aligned = all(t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 for t in (q, k, v, out))
    if q.dtype == torch.bfloat16 and aligned and _lib().af_attn_prefill_tc_supported(c_int(hd)):
        attn_prefill_tc(out, q, k, v, batch.seq_starts, batch.n_seqs, batch.max_len, nq, nkv, hd, scale, cap, window)
        return
    if (q.dtype == torch.bfloat16 and _lib().af_attn_prefill_supported(c_int(hd))
            and all(t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0 for t in (q, k, v))):
        attn_prefill_mma(out, q, k, v, batch.seq_starts, batch.n_seqs, batch.max_len, nq, nkv, hd, scale, cap, window)
        return
    attn_prefill_plain(out, q, k, v, batch.positions, nq, nkv, hd, scale, cap, window)


def attn_decode_max_splits(batch: int, nkv: int, max_len: int, window: int, blocks: int = 0, nq: int = 0) -> int:
    """The most splits the decode kernel may give one (sequence, kv head) unit:
    the room its partial results need.  The kernel's blocks (one an SM) each
    take an equal share of all units' cache pages, so a unit lies in at most
    ``blocks // units of a sequence + 2`` blocks (one long sequence among empty
    ones, whatever the batch) and in at most its pages + 1."""
    blocks = blocks or sm_count()
    rows = min(max_len, window) if window else max_len
    pages = max(1, (rows + PAGE - 1) // PAGE + (1 if window else 0))
    tiles = ((nq // nkv) + 15) // 16 if nq else 1
    return max(1, min(blocks // max(1, nkv * tiles) + 2, pages + 1))


def attn_decode_plan(page_table, slots, lens, nq: int, nkv: int, window: int, ring_rows: int, n_splits: int):
    """The plan of a decode step for :func:`attn_decode_split`: how the work is
    cut among the blocks, worked out by one small kernel for all layers that
    read the same caches the same way (these slots, lengths, page table, heads,
    window, ring and ``n_splits``).  It holds for these lengths alone."""
    lib = _lib()
    lib.af_attn_decode_plan_ints.restype = ctypes.c_longlong
    B = slots.shape[0]
    n = lib.af_attn_decode_plan_ints(c_int(B), c_int(nq), c_int(nkv))
    if n <= 0:
        raise KernelError(f"attn_decode_plan: {B} sequences, {nq} heads in {nkv} groups")
    plan = torch.empty(n, dtype=torch.int32, device=slots.device)
    _check(lib.af_attn_decode_plan(
        _ptr(plan, "plan", torch.int32), c_longlong(n), _ptr(page_table, "page_table", torch.int32),
        c_int(page_table.shape[1]), _ptr(slots, "slots", torch.int32), _ptr(lens, "lens", torch.int32), c_int(B),
        c_int(nq), c_int(nkv), c_int(window), c_int(ring_rows), c_int(n_splits), _stream()))
    return plan


def attn_decode_split(out, q, kcache, vcache, page_table, slots, lens, nq, nkv, hd, scale, cap, window, ring_rows,
                      n_splits: int, scratch=None, plan=None) -> None:
    """bfloat16 decode attention, split over the keys (two kernels: partial
    results into ``scratch``, then their merge).  ``n_splits`` is the most
    splits a (sequence, kv head) unit gets: the kernel cuts the units' pages so
    that all blocks get about the same number of them (with less room than
    :func:`attn_decode_max_splits` fewer blocks work)."""
    B = q.shape[0]
    lib = _lib()
    lib.af_attn_decode_scratch.restype = ctypes.c_longlong
    need = lib.af_attn_decode_scratch(c_int(B), c_int(nq), c_int(hd), c_int(n_splits))
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    elif scratch.numel() < need or scratch.dtype != torch.float32:
        raise KernelError(f"attn_decode_split: scratch of {need} floats wanted")
    if q.dtype != torch.bfloat16 or kcache.dtype != torch.bfloat16 or out.dtype != torch.bfloat16:
        raise KernelError("attn_decode_split: bfloat16 only")
    _check(lib.af_attn_decode(
        _ptr(out), c_longlong(_rows(out, "out")), _ptr(q), c_longlong(_rows(q, "q")), _ptr(kcache), _ptr(vcache),
        c_longlong(kcache.shape[0]), _ptr(page_table, "page_table", torch.int32), c_int(page_table.shape[1]),
        _ptr(slots, "slots", torch.int32),
        _ptr(lens, "lens", torch.int32), c_int(B), c_int(nq), c_int(nkv), c_int(hd), c_float(scale), c_float(cap),
        c_int(window), c_int(ring_rows), c_int(n_splits), _ptr(scratch, "scratch", torch.float32),
        _ptr(plan, "plan", torch.int32) if plan is not None else ctypes.c_void_p(0),
        _ptr(error_word(q.device), "err", torch.int32), _stream()))


ATTN_DECODE_MAX_SEQS = 2048     # sequences of a step that the split kernel plans for (more: the plain kernel)


def attn_decode(out, q, kv, batch, nq, nkv, hd, scale, cap, window, slopes=None) -> None:
    """Attention of a decode step over the cache: the split kernel for
    bfloat16 and head sizes it takes, else the plain kernel (which also serves
    scores with a per-head slope)."""
    if (slopes is None and q.dtype == torch.bfloat16 and _lib().af_attn_decode_supported(c_int(hd))
            and batch.n_seqs <= ATTN_DECODE_MAX_SEQS):
        n = attn_decode_max_splits(batch.n_seqs, nkv, batch.max_len_after, window, nq=nq)
        # the plan of the step, shared by the layers that read this group of caches alike (a batch without a
        # place for the step's tables gets none: every block then works the cut out itself)
        plan, aux = None, getattr(batch, "aux", None)
        if aux is not None:
            key = ("attn_decode_plan", kv.page_table.data_ptr(), kv.ring_rows, nq, nkv, window, n)
            if key not in aux:
                aux[key] = attn_decode_plan(kv.page_table, batch.slots, batch.len_after, nq, nkv, window,
                                            kv.ring_rows, n)
            plan = aux[key]
        attn_decode_split(out, q, kv.k, kv.v, kv.page_table, batch.slots, batch.len_after, nq, nkv, hd, scale, cap,
                          window, kv.ring_rows, n, plan=plan)
        return
    attn_decode_plain(out, q, kv.k, kv.v, kv.page_table, batch.slots, batch.len_after, nq, nkv, hd,
                      scale, cap, window, kv.ring_rows, slopes)




__all__ = [n for n in dir() if not n.startswith("_")]
