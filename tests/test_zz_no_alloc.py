"""The entry point that allocates nothing, called through its exported C
symbol as an embedding host would call it.

Some hosts cannot let a library allocate while they call it: all device
memory already belongs to their own pool, or allocation calls are banned in
their hot loop because they stall the device.  ``af_attn_decode_static`` is
the decode attention for them: same inputs and output as ``af_attn_decode``,
but the scratch for partial results is an array inside the library.  The test
runs it twice in a row on different inputs (the array keeps the first call's
contents; the second result must not care) and compares each result with the
existing entry point, which takes caller-owned scratch.  The file sorts last
so that a run that stops at the first failure has run every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_longlong, c_void_p

import pytest
import torch

import plain_gemma2 as plain

pytestmark = pytest.mark.gpu
PAGE = 64


def _lib():
    from airframe_b200.csrc import build
    lib = ctypes.CDLL(str(build()))
    lib.af_last_error.restype = ctypes.c_char_p
    lib.af_attn_decode_scratch.restype = c_longlong
    lib.af_attn_decode_static_capacity.restype = c_longlong
    return lib


def _problem(seed, batch, nq, nkv, hd, lens, window):
    g = torch.Generator().manual_seed(seed)
    dev = "cuda:0"
    pages_per_seq = max((n + PAGE - 1) // PAGE for n in lens)
    n_pages = batch * pages_per_seq + 2
    kc = torch.randn(n_pages, nkv, PAGE, hd, generator=g).to(torch.bfloat16).to(dev)
    vc = torch.randn(n_pages, nkv, PAGE, hd, generator=g).to(torch.bfloat16).to(dev)
    perm = torch.randperm(n_pages, generator=g)[: batch * pages_per_seq].reshape(batch, pages_per_seq)
    table = perm.to(torch.int32).to(dev)
    q = torch.randn(batch, nq * hd, generator=g).to(torch.bfloat16).to(dev)
    return dict(q=q, kc=kc, vc=vc, table=table, slots=torch.arange(batch, dtype=torch.int32, device=dev),
                lens=torch.tensor(lens, dtype=torch.int32, device=dev), window=window)


def _call(lib, fn, p, batch, nq, nkv, hd, splits, scratch=None):
    out = torch.full((batch, nq * hd), float("nan"), dtype=torch.bfloat16, device="cuda:0")
    err = torch.zeros(1, dtype=torch.int32, device="cuda:0")
    ring = ((p["window"] + PAGE - 1) // PAGE) * PAGE if p["window"] else 0
    args = [c_void_p(out.data_ptr()), c_longlong(out.stride(0)), c_void_p(p["q"].data_ptr()),
            c_longlong(p["q"].stride(0)), c_void_p(p["kc"].data_ptr()), c_void_p(p["vc"].data_ptr()),
            c_longlong(p["kc"].shape[0]), c_void_p(p["table"].data_ptr()), c_int(p["table"].shape[1]), c_void_p(p["slots"].data_ptr()),
            c_void_p(p["lens"].data_ptr()), c_int(batch), c_int(nq), c_int(nkv), c_int(hd),
            c_float(1.0 / math.sqrt(hd)), c_float(30.0), c_int(p["window"]), c_int(ring), c_int(splits)]
    if scratch is not None:
        args += [c_void_p(scratch.data_ptr()), c_void_p(0)]      # scratch of the caller's, no plan of the step
    args += [c_void_p(err.data_ptr()), c_void_p(torch.cuda.current_stream().cuda_stream)]
    rc = fn(*args)
    torch.cuda.synchronize()
    return rc, out, int(err.item())


def _plain_last_token(p, b, nq, nkv, hd, cap):
    """The plain implementation's attention of sequence b's last token over its cached rows."""
    n = int(p["lens"][b])
    pages = p["table"][b, : (n + PAGE - 1) // PAGE].long().cpu()
    k = p["kc"].cpu()[pages].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:n].double()      # [rows, kv heads, hd]
    v = p["vc"].cpu()[pages].permute(0, 2, 1, 3).reshape(-1, nkv, hd)[:n].double()
    q = torch.zeros(n, nq, hd, dtype=torch.float64)
    q[-1] = p["q"][b].cpu().double().reshape(nq, hd)
    return plain.attention(q, k, v, 1.0 / math.sqrt(hd), cap, p["window"] or None)[-1]


def test_static_scratch_entry_point_matches_the_allocating_one_twice_in_a_row():
    lib = _lib()
    batch, nq, nkv, hd, splits = 3, 8, 4, 128, 5
    need = lib.af_attn_decode_scratch(c_int(batch), c_int(nq), c_int(hd), c_int(splits))
    assert need <= lib.af_attn_decode_static_capacity() == 1 << 20
    for seed, lens, window in ((1, [300, 64, 1], 0), (2, [129, 500, 70], 0)):
        p = _problem(seed, batch, nq, nkv, hd, lens, window)
        scratch = torch.empty(need, dtype=torch.float32, device="cuda:0")
        rc_a, ref, err_a = _call(lib, lib.af_attn_decode, p, batch, nq, nkv, hd, splits, scratch)
        rc_b, got, err_b = _call(lib, lib.af_attn_decode_static, p, batch, nq, nkv, hd, splits)
        assert rc_a == 0 and rc_b == 0, lib.af_last_error()
        assert err_a == 0 and err_b == 0
        assert torch.isfinite(got.float()).all()
        diff = (got.float() - ref.float()).abs().max().item()
        assert diff <= 1.2e-2 * max(1.0, ref.float().abs().max().item()), diff    # the kernel tests' bfloat16 bound
        assert diff == 0.0                                                        # the same kernels: the same bits
        # and against the plain implementation, so that the test stands without the other entry point
        for b in range(batch):
            want = _plain_last_token(p, b, nq, nkv, hd, 30.0)
            off = (got[b].double().cpu() - want).abs().max().item()
            assert off <= 1.2e-2 * max(1.0, want.abs().max().item()), (b, off)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = _lib()
    p = _problem(3, 2, 8, 4, 256, [10, 20], 0)
    batch, nq, hd, splits = 2, 8, 256, 300                    # 2 * 8 * 300 * 258 floats > 2^20
    p_big = dict(p)
    rc, out, _ = _call(lib, lib.af_attn_decode_static, p_big, batch, nq, 4, hd, splits)
    assert rc != 0
    msg = lib.af_last_error().decode()
    assert "floats of scratch" in msg and "1048576" in msg
    assert torch.isnan(out.float()).all()                      # nothing was launched
