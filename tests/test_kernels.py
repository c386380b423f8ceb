"""Each kernel alone against the plain implementation's function for the same
part, at sizes other than the engine tests use (no power of two, head sizes
in steps of 16, odd numbers of heads and groups)."""
import math

import numpy as np
import pytest
import torch

import plain_gemma2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


@pytest.fixture(scope="module")
def K():
    from airframe_b200 import kernels
    return kernels


def tol(dtype):
    """32-bit: sums of a few thousand 32-bit products round to about sqrt(K) * 2^-24
    of the largest value (3e-6 at K = 2304): 1e-5.  bfloat16: one rounding of the
    result (2^-8) plus 32-bit sums of bfloat16 inputs: 1.2e-2."""
    return 1e-5 if dtype == torch.float32 else 1.2e-2


def close(got, ref, dtype, scale=None, k_sum=None):
    """Largest absolute error over ``scale`` (the largest reference magnitude by default;
    attention outputs use max(1, that): a bfloat16 result is off by up to one unit in its
    last place, 2^-8 of its own magnitude).  ``k_sum``: the length of the sums behind a 32-bit
    result; the bound of ``tol`` is stated for 2304 and grows with the length (the tensor cores'
    32-bit accumulators round every addition, and they round towards zero: the errors add up
    instead of cancelling)."""
    ref = ref.double()
    s = scale if scale is not None else ref.abs().max().clamp_min(1e-30)
    err = float((got.double().cpu() - ref).abs().max() / s)
    bound = tol(dtype)
    if k_sum is not None and dtype == torch.float32:
        bound *= max(1.0, k_sum / 2304)
    assert err < bound, err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed(K, dtype):
    V, H = 1000, 200
    table = torch.randn(V, H).to(dtype)
    ids = torch.tensor([0, 999, 5, 5, 321], dtype=torch.int32)
    out = torch.empty(5, H, dtype=torch.float32, device=DEV)
    K.embed(out, table.to(DEV), ids.to(DEV), math.sqrt(H))
    close(out, plain.embed(ids.tolist(), table.double(), H), torch.float32)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_and_row_gather(K, dtype):
    M, H = 7, 2304 + 48
    x = torch.randn(M, H) * 3
    w = torch.randn(H) * 0.1
    y = torch.empty(M, H, dtype=dtype, device=DEV)
    K.rmsnorm(y, x.to(DEV), w.to(DEV), 1e-5, 1.0)
    close(y, plain.rms_norm(x.double(), w.double(), 1e-5), dtype)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32)
    y2 = torch.empty(3, H, dtype=dtype, device=DEV)
    K.rmsnorm(y2, x.to(DEV), w.to(DEV), 1e-5, 1.0, rows.to(DEV))
    close(y2, plain.rms_norm(x.double()[rows.long()], w.double(), 1e-5), dtype)
    # offset 0: the weight itself multiplies (other architectures)
    K.rmsnorm(y, x.to(DEV), w.to(DEV), 1e-5, 0.0)
    close(y, plain.rms_norm(x.double(), w.double() - 1.0, 1e-5), dtype)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(K, dtype):
    M, H = 5, 1000
    x, a = torch.randn(M, H), (torch.randn(M, H) * 2).to(dtype)
    w1, w2 = torch.randn(H) * 0.1, torch.randn(H) * 0.1
    want_x = x.double() + plain.rms_norm(a.double(), w1.double(), 1e-6)
    want_y = plain.rms_norm(want_x, w2.double(), 1e-4)
    xd = x.to(DEV)
    y = torch.empty(M, H, dtype=dtype, device=DEV)
    K.add_rmsnorm(xd, a.to(DEV), w1.to(DEV), 1e-6, 1.0, y=y, w_next=w2.to(DEV), eps_next=1e-4)
    close(xd, want_x, torch.float32)
    close(y, want_y, dtype)
    xd = x.to(DEV)
    K.add_rmsnorm(xd, a.to(DEV), w1.to(DEV), 1e-6, 1.0)
    close(xd, want_x, torch.float32)
    # partial sums, added in order before the norm
    parts = torch.randn(3, M, H)
    xd = x.to(DEV)
    K.add_rmsnorm(xd, parts.to(DEV), w1.to(DEV), 1e-6, 1.0, n_parts=3)
    close(xd, x.double() + plain.rms_norm(parts.double().sum(0), w1.double(), 1e-6), torch.float32)


@pytest.mark.parametrize("H", [1024, 2304, 3584, 4608])
def test_add_rmsnorm_of_a_prompt(K, H):
    """Many rows (the variant that keeps few registers and reads the weights where it uses them)."""
    M = 300
    g = torch.Generator().manual_seed(H)
    x = torch.randn(M, H, generator=g)
    w1, w2 = torch.randn(H, generator=g) * 0.1, torch.randn(H, generator=g) * 0.1
    for a in ((torch.randn(M, H, generator=g) * 3).to(torch.bfloat16), torch.randn(2, M, H, generator=g)):
        n_parts = a.shape[0] if a.dim() == 3 else 1
        summed = a.double().sum(0) if a.dim() == 3 else a.double()
        want_x = x.double() + plain.rms_norm(summed, w1.double(), 1e-6)
        want_y = plain.rms_norm(want_x, w2.double(), 1e-5)
        xd = x.to(DEV)
        y = torch.empty(M, H, dtype=torch.bfloat16, device=DEV)
        K.add_rmsnorm(xd, a.to(DEV), w1.to(DEV), 1e-6, 1.0, y=y, w_next=w2.to(DEV), eps_next=1e-5, n_parts=n_parts)
        close(xd, want_x, torch.float32)
        close(y, want_y, torch.bfloat16)
        xd = x.to(DEV)
        K.add_rmsnorm(xd, a.to(DEV), w1.to(DEV), 1e-6, 1.0, n_parts=n_parts)
        close(xd, want_x, torch.float32)


@pytest.mark.parametrize("H", [1100, 2304, 4608])
@pytest.mark.parametrize("n_parts", [1, 3, 9])
def test_add_rmsnorm_of_a_decode_step(K, H, n_parts):
    """Few rows of many 32-bit partial sums, as a decode step has them; one row's result does not depend
    on the others."""
    M = 7
    g = torch.Generator().manual_seed(H + n_parts)
    x = torch.randn(M, H, generator=g)
    parts = torch.randn(n_parts, M, H, generator=g) * 2
    parts[:, 3] *= 30.0                                    # a row with another scale
    w1, w2 = torch.randn(H, generator=g) * 0.1, torch.randn(H, generator=g) * 0.1
    want_x = x.double() + plain.rms_norm(parts.double().sum(0), w1.double(), 1e-6)
    want_y = plain.rms_norm(want_x, w2.double(), 1e-5)
    for ydt in (torch.bfloat16, torch.float32):
        xd = x.to(DEV)
        y = torch.empty(M, H, dtype=ydt, device=DEV)
        K.add_rmsnorm(xd, parts.to(DEV), w1.to(DEV), 1e-6, 1.0, y=y, w_next=w2.to(DEV), eps_next=1e-5, n_parts=n_parts)
        close(xd, want_x, torch.float32)
        close(y, want_y, ydt)
    xd1 = x.to(DEV)
    K.add_rmsnorm(xd1, parts.to(DEV), w1.to(DEV), 1e-6, 1.0, n_parts=n_parts)     # without a next norm
    close(xd1, want_x, torch.float32)
    # rows alone give the same bits as rows together
    x3 = x[3:4].to(DEV)
    K.add_rmsnorm(x3, parts[:, 3:4].contiguous().to(DEV), w1.to(DEV), 1e-6, 1.0, n_parts=n_parts)
    assert torch.equal(x3[0], xd1[3])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_act(K, dtype):
    M, I = 3, 1111
    gu = (torch.randn(M, 2 * I) * 2).to(dtype)
    out = torch.empty(M, I, dtype=dtype, device=DEV)
    K.gated_act(out, gu.to(DEV), "gelu_tanh")
    g, u = gu.double()[:, :I], gu.double()[:, I:]
    close(out, plain.gelu_tanh(g) * u, dtype)
    K.gated_act(out, gu.to(DEV), "silu")
    close(out, g * torch.sigmoid(g) * u, dtype)
    with pytest.raises(K.KernelError, match="unknown activation"):
        K.gated_act(out, gu.to(DEV), "relu")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(1, 130, 70), (5, 64, 16), (67, 129, 257), (3, 1000, 2304)])
def test_gemm_plain(K, dtype, shape):
    M, N, Kd = shape
    x, w = torch.randn(M, Kd).to(dtype), (torch.randn(N, Kd) * 0.05).to(dtype)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    K.gemm_plain(out, x.to(DEV), w.to(DEV))
    ref = x.double() @ w.double().T
    close(out, ref, dtype)
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    K.gemm_plain(out32, x.to(DEV), w.to(DEV), cap=2.0)
    close(out32, plain.softcap(ref, 2.0), torch.float32)


def test_gemm_plain_is_true_32_bit_and_batch_invariant(K):
    """Values that a reduced-precision product would lose; and a row's result
    does not change with the rows around it."""
    x = torch.tensor([[1.0, 2 ** -20, -1.0]])
    w = torch.tensor([[1.0, 1.0, 1.0]])
    out = torch.empty(1, 1, dtype=torch.float32, device=DEV)
    K.gemm_plain(out, x.to(DEV), w.to(DEV))
    assert out.item() == 2 ** -20
    x = torch.randn(70, 300)
    w = torch.randn(90, 300)
    a = torch.empty(70, 90, device=DEV)
    b = torch.empty(1, 90, device=DEV)
    K.gemm_plain(a, x.to(DEV), w.to(DEV))
    K.gemm_plain(b, x[37:38].to(DEV), w.to(DEV))
    assert torch.equal(a[37], b[0])


def _paged(k, v, order, n_pages, dtype):
    """Scatter k, v [T, nkv, hd] of one sequence into pages in the given order."""
    T, nkv, hd = k.shape
    kc = torch.zeros(n_pages, nkv, PAGE, hd, dtype=dtype)
    vc = torch.zeros(n_pages, nkv, PAGE, hd, dtype=dtype)
    for r in range(T):
        p = order[r // PAGE]
        kc[p, :, r % PAGE] = k[r]
        vc[p, :, r % PAGE] = v[r]
    return kc, vc


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("pairing,rot", [("half", 48), ("half", 32), ("adjacent", 48)])
def test_rope_and_cache_write(K, dtype, pairing, rot):
    nq, nkv, hd, theta = 3, 1, 48, 5000.0
    lens = [70, 3]                                    # two sequences, rows concatenated
    T = sum(lens)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd).to(dtype)
    pos = torch.tensor(list(range(70)) + list(range(3)), dtype=torch.int32)
    seq = torch.tensor([0] * 70 + [1] * 3, dtype=torch.int32)
    inv = (torch.tensor(theta, dtype=torch.float64) ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    table = torch.tensor([[5, 2, -1], [0, -1, -1], [1, 1, 1]], dtype=torch.int32)   # slot -> pages
    slots = torch.tensor([0, 1], dtype=torch.int32)
    kc = torch.zeros(6, nkv, PAGE, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    d = qkv.to(DEV)
    K.rope_cache_write(d, pos.to(DEV), inv.to(DEV), nq, nkv, hd, rot, pairing, seq_of_token=seq.to(DEV),
                       slots=slots.to(DEV), len_after=torch.tensor(lens, dtype=torch.int32, device=DEV),
                       kcache=kc, vcache=vc, page_table=table.to(DEV), ring_rows=0)
    x = qkv.double().reshape(T, nq + 2 * nkv, hd)

    def rotate(h):                                     # [T, heads, hd] with the plain rope on the rotary part
        part = h[..., :rot]
        if pairing == "adjacent":                      # (2p, 2p+1) pairs -> half layout and back
            part = torch.cat([part[..., 0::2], part[..., 1::2]], -1)
        r = plain.rope(part, pos.tolist(), theta)
        if pairing == "adjacent":
            out = torch.empty_like(r)
            out[..., 0::2], out[..., 1::2] = r[..., : rot // 2], r[..., rot // 2:]
            r = out
        return torch.cat([r, h[..., rot:]], -1)

    want = torch.cat([rotate(x[:, : nq + nkv]), x[:, nq + nkv:]], 1)
    close(d.reshape(T, -1, hd), want, dtype)
    got_k = torch.cat([kc[5, :, :, :].cpu(), kc[2, :, :6].cpu()], 1).transpose(0, 1)       # rows 0..69 of slot 0
    close(got_k, want[:70, nq: nq + nkv], dtype)
    close(vc[0, :, :3].cpu().transpose(0, 1), want[70:, nq + nkv:], dtype)
    assert float(kc[1].abs().sum()) == 0 and float(kc[2, :, 6:].abs().sum()) == 0          # nothing else touched


@pytest.mark.parametrize("hd,nq,nkv,Kd,lens,ring", [
    (64, 3, 1, 72, [70, 3], 0),              # one tile and a half of weight rows, a single small token tile
    (256, 2, 1, 264, [5], 0),                # head size 256: a head is two weight tiles
    (128, 4, 2, 2304, [8, 1, 7], 0),         # few tokens and a long K: split-K, the last block adds the parts
    (96, 2, 2, 520, [40, 9], 0),             # head size 96: three groups of pairs a head
    (256, 8, 4, 136, [300], 128),            # many tokens (two accumulators), a ring that the prompt laps
    (32, 5, 5, 64, [130, 2, 64], 64)])
def test_projection_with_rotary_and_cache_write_in_its_epilogue(K, hd, nq, nkv, Kd, lens, ring):
    theta = 10000.0
    T, B = sum(lens), len(lens)
    N = (nq + 2 * nkv) * hd
    g = torch.Generator().manual_seed(hd + T)
    x = torch.randn(T, Kd, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, Kd, generator=g) * 0.08).to(torch.bfloat16)
    pos = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32)
    seq = torch.tensor([b for b, n in enumerate(lens) for _ in range(n)], dtype=torch.int32)
    inv = (torch.tensor(theta, dtype=torch.float64) ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float()
    pages_per = max((min(n, ring) if ring else n) + PAGE - 1 for n in lens) // PAGE
    n_pages = B * pages_per + 1
    perm = torch.randperm(n_pages - 1, generator=g)[: B * pages_per].reshape(B, pages_per) + 1   # page 0 stays unused
    kc = torch.zeros(n_pages, nkv, PAGE, hd, dtype=torch.bfloat16, device=DEV)
    vc = torch.zeros_like(kc)

    class Batch:
        tokens = torch.zeros(T, dtype=torch.int32, device=DEV)
        positions = pos.to(DEV)
        seq_of_token = seq.to(DEV)
        slots = torch.arange(B, dtype=torch.int32, device=DEV)
        len_after = torch.tensor(lens, dtype=torch.int32, device=DEV)

    class View:
        k, v = kc, vc
        page_table = perm.to(torch.int32).to(DEV)
        ring_rows = ring

    table = K.rope_table(Batch.positions, inv.to(DEV))
    ang = pos.double()[:, None] * inv.double()[None, :]
    assert float((table[..., 0].cpu().double() - torch.cos(ang)).abs().max()) < 2e-3      # 32-bit angles of positions to 300
    rows = K.kv_rows(Batch, View, nkv)
    order = K.rope_row_order(nq + 2 * nkv, hd)
    assert sorted(order.tolist()) == list(range(N))
    wp = w[order].contiguous().to(DEV)
    # the reference: the plain product, the plain rotation of q and k heads
    y = (x.double() @ w.double().T).reshape(T, nq + 2 * nkv, hd)
    want = torch.cat([plain.rope(y[:, : nq + nkv], pos.tolist(), theta), y[:, nq + nkv:]], 1)
    splits = K.gemm_tc_splits(T, N, Kd) if T <= 64 else 1
    tickets = torch.zeros(4 * ((N + 127) // 128), dtype=torch.int32, device=DEV)
    for attempt in range(2):                          # twice: the tickets must come back to zero
        out = torch.full((T, N), float("nan"), dtype=torch.bfloat16, device=DEV)
        kc.zero_(), vc.zero_()
        K.gemm_tc_rope(out, x.to(DEV), wp, table, nq, nkv, hd, rows, kc, vc, splits=splits, tickets=tickets)
        K.check_device_errors(DEV)
        assert int(tickets.abs().sum()) == 0
        close(out.reshape(T, -1, hd), want, torch.bfloat16)
        # the cache holds, for every sequence, the rows that a ring keeps (all rows without one)
        first = 0
        for b, n in enumerate(lens):
            for p_ in range(max(0, n - ring) if ring else 0, n):
                r = p_ % ring if ring else p_
                page = int(perm[b, r // PAGE])
                got_k, got_v = kc[page, :, r % PAGE].cpu(), vc[page, :, r % PAGE].cpu()
                assert torch.equal(got_k, out[first + p_].reshape(-1, hd)[nq: nq + nkv].cpu()), (b, p_)
                assert torch.equal(got_v, out[first + p_].reshape(-1, hd)[nq + nkv:].cpu()), (b, p_)
            first += n
        assert float(kc[0].abs().sum()) == 0                       # a page of no sequence stays untouched
    if splits > 1:
        # the sum of the partial tiles does not depend on which block came last: the same bits every time
        again = torch.empty_like(out)
        K.gemm_tc_rope(again, x.to(DEV), wp, table, nq, nkv, hd, rows, kc, vc, splits=splits, tickets=tickets)
        assert torch.equal(again, out)
    # without a cache nothing is stored
    kc.zero_()
    K.gemm_tc_rope(out, x.to(DEV), wp, table, nq, nkv, hd, splits=splits, tickets=tickets)
    assert float(kc.abs().sum()) == 0
    with pytest.raises(K.KernelError, match="multiple of 32"):
        K.rope_row_order(3, 48)


def test_ring_keeps_the_last_rows_of_a_long_prompt(K):
    nq, nkv, hd = 1, 1, 16
    T, ring = 150, 128
    qkv = torch.randn(T, 3 * hd)
    pos = torch.arange(T, dtype=torch.int32)
    table = torch.tensor([[3, 1]], dtype=torch.int32)
    kc = torch.zeros(4, nkv, PAGE, hd, device=DEV)
    vc = torch.zeros_like(kc)
    K.rope_cache_write(qkv.to(DEV), pos.to(DEV), torch.zeros(0, device=DEV), nq, nkv, hd, 0, "half",
                       seq_of_token=torch.zeros(T, dtype=torch.int32, device=DEV),
                       slots=torch.zeros(1, dtype=torch.int32, device=DEV),
                       len_after=torch.tensor([T], dtype=torch.int32, device=DEV), kcache=kc, vcache=vc,
                       page_table=table.to(DEV), ring_rows=ring)
    v = qkv[:, 2 * hd:]
    for p in range(T - ring, T):                       # positions 22..149 live in row p % 128
        r = p % ring
        page = [3, 1][r // PAGE]
        assert torch.equal(vc[page, 0, r % PAGE].cpu(), v[p]), p


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,nq,nkv,window,cap", [(16, 4, 2, 0, 50.0), (80, 6, 2, 7, 0.0), (256, 3, 3, 33, 30.0),
                                                  (48, 5, 1, 0, 20.0)])
def test_attention_prefill_plain(K, dtype, hd, nq, nkv, window, cap):
    torch.manual_seed(hd + nq + window)               # (unseeded inputs once met the bound's edge: outputs of magnitude 4)
    lens = [37, 1, 90]
    T = sum(lens)
    q = torch.randn(T, nq * hd).to(dtype)
    k = torch.randn(T, nkv * hd).to(dtype)
    v = torch.randn(T, nkv * hd).to(dtype)
    pos = torch.tensor([p for n in lens for p in range(n)], dtype=torch.int32)
    out = torch.empty(T, nq * hd, dtype=dtype, device=DEV)
    scale = 0.7 / math.sqrt(hd)
    K.attn_prefill_plain(out, q.to(DEV), k.to(DEV), v.to(DEV), pos.to(DEV), nq, nkv, hd, scale, cap, window)
    o = 0
    for n in lens:
        ref = plain.attention(q[o:o + n].double().reshape(n, nq, hd), k[o:o + n].double().reshape(n, nkv, hd),
                              v[o:o + n].double().reshape(n, nkv, hd), scale, cap, window or None)
        close(out[o:o + n], ref, dtype, scale=max(1.0, float(ref.abs().max())))
        o += n


def _decode_case(K, dtype, hd, nq, nkv, window, cap, lens, q, ks, vs, scale, n_splits=None, padding=(), plan=False):
    """Sequences with their own lengths in permuted pages; returns kernel output [B, nq*hd].  ``n_splits``: the
    split kernel with that much room for partial results; ``padding``: rows of the batch without a slot;
    ``plan``: the cut comes from the step's plan (else every block works it out itself)."""
    B = len(lens)
    ring = ((window + PAGE - 1) // PAGE) * PAGE if window else 0
    per_seq = max(((min(n, ring) if ring else n) + PAGE - 1) // PAGE for n in lens)
    n_pages = B * per_seq + 3
    perm = torch.randperm(n_pages).tolist()
    table = torch.full((B + 2, per_seq), -1, dtype=torch.int32)
    kc = torch.zeros(n_pages, nkv, PAGE, hd, dtype=dtype)
    vc = torch.zeros_like(kc)
    slots = [B + 1 - b for b in range(B)]              # slots are not the batch order
    for b, n in enumerate(lens):
        for r_pos in range(n):
            if ring and r_pos + ring < n:
                continue
            r = r_pos % ring if ring else r_pos
            if table[slots[b], r // PAGE] < 0:
                table[slots[b], r // PAGE] = perm.pop()
            p = int(table[slots[b], r // PAGE])
            kc[p, :, r % PAGE] = ks[b][r_pos]
            vc[p, :, r % PAGE] = vs[b][r_pos]
    out = torch.full((B, nq * hd), float("nan"), dtype=dtype, device=DEV)
    slots_t = torch.tensor([-1 if b in padding else sl for b, sl in enumerate(slots)], dtype=torch.int32, device=DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
    if n_splits is not None:
        table_d = table.to(DEV)
        the_plan = K.attn_decode_plan(table_d, slots_t, lens_t, nq, nkv, window, ring, n_splits) if plan else None
        K.attn_decode_split(out, q.to(DEV), kc.to(DEV), vc.to(DEV), table_d, slots_t, lens_t, nq, nkv, hd,
                            scale, cap, window, ring, n_splits, plan=the_plan)
        return out
    batch = _Batch(slots_t, lens_t, max(lens))
    if plan:
        batch.aux = {}
    K.attn_decode(out, q.to(DEV), _View(kc.to(DEV), vc.to(DEV), table.to(DEV), ring), batch, nq, nkv, hd, scale, cap,
                  window)
    if plan and dtype == torch.bfloat16 and hd in (64, 128, 256):
        assert any(k[0] == "attn_decode_plan" for k in batch.aux)
    return out


class _View:
    def __init__(self, k, v, table, ring):
        self.k, self.v, self.page_table, self.ring_rows = k, v, table, ring


class _Batch:
    def __init__(self, slots, len_after, max_len_after):
        self.slots, self.len_after, self.max_len_after = slots, len_after, max_len_after
        self.n_seqs = slots.shape[0]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,nq,nkv,window,cap", [(16, 4, 2, 0, 50.0), (80, 6, 2, 70, 0.0), (256, 8, 4, 100, 50.0),
                                                  (128, 5, 5, 0, 30.0), (48, 6, 1, 64, 0.0)])
def test_attention_decode_over_pages(K, dtype, hd, nq, nkv, window, cap):
    torch.manual_seed(hd + nq)
    lens = [1, 64, 65, 300, 129]
    scale = 1.3 / math.sqrt(hd)
    q = torch.randn(len(lens), nq * hd).to(dtype)
    ks = [torch.randn(n, nkv, hd).to(dtype) for n in lens]
    vs = [torch.randn(n, nkv, hd).to(dtype) for n in lens]
    out = _decode_case(K, dtype, hd, nq, nkv, window, cap, lens, q, ks, vs, scale)
    for b, n in enumerate(lens):
        # the new token is the last row: build a whole-sequence problem whose last query is q[b]
        qq = torch.zeros(n, nq, hd, dtype=torch.float64)
        qq[-1] = q[b].double().reshape(nq, hd)
        ref = plain.attention(qq, ks[b].double(), vs[b].double(), scale, cap, window or None)[-1]
        close(out[b], ref, dtype, scale=1.0)


@pytest.mark.parametrize("plan", [False, True])
@pytest.mark.parametrize("hd,nq,nkv,window", [(256, 8, 4, 0), (128, 6, 2, 0), (256, 4, 2, 300), (128, 16, 2, 1000)])
def test_attention_decode_one_long_sequence_among_short_ones(K, hd, nq, nkv, window, plan):
    """The split kernel cuts every sequence by its own length: the long one into many splits, the short
    ones into one; a key far back in the long one has to be found."""
    dtype = torch.bfloat16
    torch.manual_seed(hd + window)
    lens = [3, 2500, 70, 1, 640, 129, 64]
    scale = 1.0 / math.sqrt(hd)
    q = torch.randn(len(lens), nq * hd).to(dtype)
    ks = [(torch.randn(n, nkv, hd) * 0.3).to(dtype) for n in lens]
    vs = [torch.randn(n, nkv, hd).to(dtype) for n in lens]
    far = 2500 - 1 - (150 if window else 2100)
    ks[1][far] = (q[1].float().reshape(nq, hd)[: nq // nkv].sum(0) * 6.0).to(dtype)     # the first kv group's heads score it high
    out = _decode_case(K, dtype, hd, nq, nkv, window, 30.0, lens, q, ks, vs, scale, plan=plan)
    for b, n in enumerate(lens):
        qq = torch.zeros(n, nq, hd, dtype=torch.float64)
        qq[-1] = q[b].double().reshape(nq, hd)
        ref = plain.attention(qq, ks[b].double(), vs[b].double(), scale, 30.0, window or None)[-1]
        close(out[b], ref, dtype, scale=1.0)
    near = (out[1].double().cpu().reshape(nq, hd)[0] - vs[1][far, 0].double()).abs().max()
    assert near < 0.1, float(near)


def _check_decode(K, out, lens, q, ks, vs, nq, hd, scale, cap, window, padding=()):
    for b, n in enumerate(lens):
        if b in padding:
            assert float(out[b].float().abs().max()) == 0.0, b          # a row without a slot gives zeros
            continue
        qq = torch.zeros(n, nq, hd, dtype=torch.float64)
        qq[-1] = q[b].double().reshape(nq, hd)
        ref = plain.attention(qq, ks[b].double(), vs[b].double(), scale, cap, window or None)[-1]
        close(out[b], ref, torch.bfloat16, scale=1.0)


@pytest.mark.parametrize("plan", [False, True])
@pytest.mark.parametrize("hd,nq,nkv,window", [(256, 8, 4, 0), (128, 8, 4, 200), (64, 40, 2, 0), (128, 12, 2, 0)])
def test_attention_decode_many_short_sequences_share_blocks(K, hd, nq, nkv, window, plan):
    """More (sequence, kv head) units than blocks: the blocks take equal runs of the units' pages end to end, so a
    block ends one unit and begins the next (other sequence, other kv head, other tile of heads) and leaves a
    partial result for each.  Rows without a slot lie between them.  (40 heads in 2 groups: tiles of 16 and 4.)"""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(hd + nq)
    n_seq = 90 if nkv == 2 else 50
    lens = [int(x) for x in torch.randint(1, 330, (n_seq,), generator=g)]
    lens[3], lens[17] = 1, 64
    padding = (0, 5, 6, n_seq - 1)
    scale = 1.0 / math.sqrt(hd)
    q = torch.randn(n_seq, nq * hd, generator=g).to(dtype)
    ks = [(torch.randn(n, nkv, hd, generator=g) * 0.5).to(dtype) for n in lens]
    vs = [torch.randn(n, nkv, hd, generator=g).to(dtype) for n in lens]
    out = _decode_case(K, dtype, hd, nq, nkv, window, 30.0, lens, q, ks, vs, scale, padding=padding, plan=plan)
    _check_decode(K, out, lens, q, ks, vs, nq, hd, scale, 30.0, window, padding)


@pytest.mark.parametrize("plan", [False, True])
@pytest.mark.parametrize("n_splits", [1, 2, 3, 5, 9, 64])
def test_attention_decode_with_any_room_for_partial_results(K, n_splits, plan):
    """The caller says how many partial results a unit may leave; with little room fewer blocks work, and the
    result is the same."""
    dtype, hd, nq, nkv = torch.bfloat16, 128, 6, 2
    torch.manual_seed(n_splits)
    lens = [700, 3, 1500, 64, 200, 129, 2000, 90, 1, 333, 65, 1000]
    scale = 1.0 / math.sqrt(hd)
    q = torch.randn(len(lens), nq * hd).to(dtype)
    ks = [(torch.randn(n, nkv, hd) * 0.5).to(dtype) for n in lens]
    vs = [torch.randn(n, nkv, hd).to(dtype) for n in lens]
    out = _decode_case(K, dtype, hd, nq, nkv, 0, 0.0, lens, q, ks, vs, scale, n_splits=n_splits, plan=plan)
    _check_decode(K, out, lens, q, ks, vs, nq, hd, scale, 0.0, 0)


def test_attention_decode_one_sequence_in_many_splits(K):
    """One sequence alone is cut into a split a page (more than the merge's short path takes): a key in the
    first page and one in the last both count."""
    dtype, hd, nq, nkv, n = torch.bfloat16, 256, 8, 4, 4000
    torch.manual_seed(11)
    q = torch.randn(1, nq * hd).to(dtype)
    k = (torch.randn(n, nkv, hd) * 0.05).to(dtype)
    v = torch.randn(n, nkv, hd).to(dtype)
    qv = q.float().reshape(nq, hd)
    k[7, 0] = (qv[0] * 4.0).to(dtype)
    k[n - 2, 0] = (qv[0] * 4.0).to(dtype)
    scale = 1.0 / math.sqrt(hd)
    out = _decode_case(K, dtype, hd, nq, nkv, 0, 0.0, [n], q, [k], [v], scale)
    _check_decode(K, out, [n], q, [k], [v], nq, hd, scale, 0.0, 0)
    both = 0.5 * (v[7, 0].double() + v[n - 2, 0].double())
    assert float((out[0].double().cpu().reshape(nq, hd)[0] - both).abs().max()) < 0.1
    assert K.attn_decode_max_splits(1, nkv, n, 0, nq=nq) > 8


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_finds_one_far_key_and_the_window_edge(K, dtype):
    """Random keys would hide a lost row among hundreds: one key is made to
    dominate, first far back, then exactly at and just outside the window's edge."""
    hd, nq, nkv, n = 64, 2, 1, 700
    torch.manual_seed(3)
    q = torch.randn(1, nq * hd).to(dtype)
    base_k = torch.randn(n, nkv, hd) * 0.01
    v = torch.randn(n, nkv, hd).to(dtype)
    qv = q.double().reshape(nq, hd)
    for window, far in [(0, 5), (0, 333), (257, n - 257), (257, n - 258), (64, n - 64), (64, n - 65)]:
        k = base_k.clone()
        k[far, 0] = (qv[0] + qv[1]).float() * 8.0          # both heads score it high
        k = k.to(dtype)
        out = _decode_case(K, dtype, hd, nq, nkv, window, 0.0, [n], q, [k], [v], 1.0)
        visible = window == 0 or (n - 1 - far) < window
        qq = torch.zeros(n, nq, hd, dtype=torch.float64)
        qq[-1] = qv
        ref = plain.attention(qq, k.double(), v.double(), 1.0, 0.0, window or None)[-1]
        close(out[0], ref, dtype, scale=1.0)
        near = (out[0].double().cpu().reshape(nq, hd) - v[far, 0].double()).abs().max()
        assert (near < 0.05) == visible, (window, far, float(near))


def test_kernels_refuse_what_they_cannot_do(K):
    x = torch.zeros(2, 4)
    with pytest.raises(K.KernelError, match="CUDA device"):
        K.rmsnorm(x, x, x[0], 1e-6, 1.0)
    with pytest.raises(K.KernelError, match="float32 or bfloat16"):
        K.dtype_code(torch.float16)
    q = torch.zeros(1, 528, device=DEV)
    with pytest.raises(K.KernelError, match="head_dim 528"):
        K.attn_prefill_plain(q, q, q, q, torch.zeros(1, dtype=torch.int32, device=DEV), 1, 1, 528, 1.0, 0.0, 0)
    with pytest.raises(K.KernelError, match="heads 3, groups 2"):
        K.attn_prefill_plain(q, q, q, q, torch.zeros(1, dtype=torch.int32, device=DEV), 3, 2, 16, 1.0, 0.0, 0)


@pytest.mark.parametrize("M,N,Kd", [(1, 128, 64), (8, 256, 128), (5, 130, 72), (16, 2304, 2304), (33, 384, 200),
                                    (64, 100, 1000), (100, 640, 328), (300, 384, 264), (700, 130, 2048),
                                    (520, 6400, 136)])      # the last: more tiles than SMs, a block walks several
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tensor_cores(K, M, N, Kd, out_dtype):
    torch.manual_seed(M * N + Kd)
    x = torch.randn(M, Kd).to(torch.bfloat16)
    w = (torch.randn(N, Kd) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    for n_acc in (0, 1, 2, 4):                        # 4: the kernel on pairs of SMs
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        K.gemm_tc(out, x.to(DEV), w.to(DEV), n_acc=n_acc)
        K.check_device_errors(DEV)
        close(out, ref, out_dtype if out_dtype == torch.bfloat16 else torch.float32)
    if out_dtype == torch.float32:
        out.fill_(float("nan"))
        K.gemm_tc(out, x.to(DEV), w.to(DEV), cap=1.5, n_acc=4)
        close(out, plain.softcap(ref, 1.5), torch.float32)
        K.gemm_tc(out, x.to(DEV), w.to(DEV), cap=1.5)
        close(out, plain.softcap(ref, 1.5), torch.float32)
        # against the plain kernel on the same inputs: only the order of the 32-bit sums differs
        twin = torch.empty(M, N, dtype=torch.float32, device=DEV)
        K.gemm_plain(twin, x.to(DEV), w.to(DEV), cap=1.5)
        close(out, twin.cpu(), torch.float32)


@pytest.mark.parametrize("M,N,Kd", [(2048, 2304, 2304), (16384, 384, 520), (2048, 300, 9216), (4100, 18432 // 16, 264)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tensor_cores_many_token_tiles(K, M, N, Kd, out_dtype):
    """Prompts of thousands of tokens: 8 to 64 token tiles, which the blocks walk tile after tile."""
    torch.manual_seed(M + N + Kd)
    x = torch.randn(M, Kd).to(torch.bfloat16)
    w = (torch.randn(N, Kd) * 0.05).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    for n_acc in (0, 1, 2, 4):
        out = torch.full((M, N), float("nan"), dtype=out_dtype, device=DEV)
        K.gemm_tc(out, x.to(DEV), w.to(DEV), n_acc=n_acc)
        K.check_device_errors(DEV)
        close(out, ref, out_dtype if out_dtype == torch.bfloat16 else torch.float32, k_sum=Kd)


@pytest.mark.parametrize("M,N,Kd,splits", [(8, 256, 1024, 4), (3, 130, 2304, 9), (40, 384, 9216, 16), (16, 128, 520, 3)])
def test_gemm_tensor_cores_split_k(K, M, N, Kd, splits):
    x = torch.randn(M, Kd).to(torch.bfloat16)
    w = (torch.randn(N, Kd) * 0.05).to(torch.bfloat16)
    out = torch.full((splits, M, N), float("nan"), dtype=torch.float32, device=DEV)
    K.gemm_tc(out, x.to(DEV), w.to(DEV), splits=splits)
    K.check_device_errors(DEV)
    close(out.sum(0), x.double() @ w.double().T, torch.float32)
    assert 1 <= K.gemm_tc_splits(8, 2304, 9216) <= 16 and K.gemm_tc_splits(8, 256000, 2304) == 1


@pytest.mark.parametrize("M,I,Kd,act", [(8, 256, 128, "gelu_tanh"), (5, 200, 72, "silu"), (130, 448, 192, "gelu_tanh"),
                                        (300, 9216, 2304, "gelu_tanh"), (40, 64, 64, "silu")])
def test_gemm_tensor_cores_gated(K, M, I, Kd, act):
    x = torch.randn(M, Kd).to(torch.bfloat16)
    w = (torch.randn(2 * I, Kd) * 0.05).to(torch.bfloat16)
    g = x.double() @ w[:I].double().T
    u = x.double() @ w[I:].double().T
    ref = (plain.gelu_tanh(g) if act == "gelu_tanh" else g * torch.sigmoid(g)) * u
    wi = K.interleave_gate_up(w[:I].to(DEV), w[I:].to(DEV))
    assert wi.shape[0] == (I + 15) // 16 * 32 and torch.equal(wi[16:32].cpu(), w[I: I + 16])
    for n_acc in (1, 2, 4):
        out = torch.full((M, wi.shape[0] // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
        K.gemm_tc(out, x.to(DEV), wi, gated=True, activation=act, n_acc=n_acc)
        K.check_device_errors(DEV)
        close(out[:, :I], ref, torch.bfloat16)


def test_gemm_tensor_cores_refuses_unaligned(K):
    x = torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 12, dtype=torch.bfloat16, device=DEV)
    assert not K.gemm_tc_supported(x, w, None)
    with pytest.raises(K.KernelError, match="K % 8"):
        K.gemm_tc(torch.zeros(4, 8, dtype=torch.bfloat16, device=DEV), x, w)


@pytest.mark.parametrize("hd,nq,nkv,window,cap", [(64, 4, 2, 0, 50.0), (128, 6, 2, 70, 0.0), (256, 4, 2, 300, 30.0),
                                                  (256, 2, 1, 0, 0.0), (64, 3, 3, 5, 20.0), (128, 2, 2, 64, 10.0)])
def test_attention_prefill_tensor_cores(K, hd, nq, nkv, window, cap):
    torch.manual_seed(hd + window)
    lens = [37, 1, 200, 128, 129, 64, 513]
    T = sum(lens)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd).to(torch.bfloat16).to(DEV)      # packed rows, as the mixer holds them
    q, k, v = qkv[:, : nq * hd], qkv[:, nq * hd: (nq + nkv) * hd], qkv[:, (nq + nkv) * hd:]
    starts = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    scale = 1.1 / math.sqrt(hd)
    K.attn_prefill_mma(out, q, k, v, starts, len(lens), max(lens), nq, nkv, hd, scale, cap, window)
    o = 0
    for n in lens:
        ref = plain.attention(q[o:o + n].double().cpu().reshape(n, nq, hd), k[o:o + n].double().cpu().reshape(n, nkv, hd),
                              v[o:o + n].double().cpu().reshape(n, nkv, hd), scale, cap, window or None)
        close(out[o:o + n], ref, torch.bfloat16, scale=1.0)
        o += n


def test_attention_prefill_tensor_cores_finds_one_far_key_and_the_window_edge(K):
    hd, nq, nkv, n = 128, 2, 1, 700
    torch.manual_seed(4)
    q = (torch.randn(n, nq * hd) * 0.05)
    base_k = torch.randn(n, nkv * hd) * 0.01
    v = torch.randn(n, nkv * hd).to(torch.bfloat16)
    starts = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    row = n - 1
    qv = torch.randn(nq, hd)
    q[row] = qv.reshape(-1)
    for window, far in [(0, 5), (0, 333), (257, row - 256), (257, row - 257), (64, row - 63), (64, row - 64)]:
        k = base_k.clone()
        k[far] = (qv[0] + qv[1]) * 8.0
        qb, kb = q.to(torch.bfloat16), k.to(torch.bfloat16)
        out = torch.empty(n, nq * hd, dtype=torch.bfloat16, device=DEV)
        K.attn_prefill_mma(out, qb.to(DEV), kb.to(DEV), v.to(DEV), starts, 1, n, nq, nkv, hd, 1.0, 0.0, window)
        ref = plain.attention(qb.double().reshape(n, nq, hd), kb.double().reshape(n, nkv, hd),
                              v.double().reshape(n, nkv, hd), 1.0, 0.0, window or None)
        close(out, ref, torch.bfloat16, scale=1.0)
        visible = window == 0 or (row - far) < window
        near = (out[row].double().cpu().reshape(nq, hd) - v[far].double()).abs().max()
        assert (near < 0.05) == visible, (window, far, float(near))


@pytest.mark.parametrize("hd,nq,nkv,window,cap", [(128, 6, 2, 70, 0.0), (256, 4, 2, 300, 30.0), (256, 2, 1, 0, 0.0),
                                                  (128, 2, 2, 64, 10.0), (256, 8, 4, 0, 50.0), (128, 3, 1, 5, 20.0)])
def test_attention_prefill_tcgen05(K, hd, nq, nkv, window, cap):
    torch.manual_seed(hd + window)
    lens = [37, 1, 200, 128, 129, 64, 513, 1000]
    T = sum(lens)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd).to(torch.bfloat16).to(DEV)      # packed rows, as the mixer holds them
    q, k, v = qkv[:, : nq * hd], qkv[:, nq * hd: (nq + nkv) * hd], qkv[:, (nq + nkv) * hd:]
    starts = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
    out = torch.full((T, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    scale = 1.1 / math.sqrt(hd)
    K.attn_prefill_tc(out, q, k, v, starts, len(lens), max(lens), nq, nkv, hd, scale, cap, window)
    K.check_device_errors(DEV)
    o = 0
    for n in lens:
        ref = plain.attention(q[o:o + n].double().cpu().reshape(n, nq, hd), k[o:o + n].double().cpu().reshape(n, nkv, hd),
                              v[o:o + n].double().cpu().reshape(n, nkv, hd), scale, cap, window or None)
        close(out[o:o + n], ref, torch.bfloat16, scale=max(1.0, float(ref.abs().max())))
        o += n
    # the twin on the legacy tensor path sees the same inputs
    twin = torch.empty_like(out)
    K.attn_prefill_mma(twin, q, k, v, starts, len(lens), max(lens), nq, nkv, hd, scale, cap, window)
    close(out, twin.double().cpu(), torch.bfloat16, scale=max(1.0, float(twin.float().abs().max())))


def test_attention_prefill_tcgen05_finds_one_far_key_the_window_edge_and_a_growing_maximum(K):
    """One dominant key far back, at and just outside the window's edge; and scores that grow
    along the sequence, so that the reference maximum has to move and O is rescaled."""
    hd, nq, nkv, n = 128, 2, 1, 700
    torch.manual_seed(4)
    q = (torch.randn(n, nq * hd) * 0.05)
    base_k = torch.randn(n, nkv * hd) * 0.01
    v = torch.randn(n, nkv * hd).to(torch.bfloat16)
    starts = torch.tensor([0, n], dtype=torch.int32, device=DEV)
    row = n - 1
    qv = torch.randn(nq, hd)
    q[row] = qv.reshape(-1)
    for window, far in [(0, 5), (0, 333), (257, row - 256), (257, row - 257), (64, row - 63), (64, row - 64)]:
        k = base_k.clone()
        k[far] = (qv[0] + qv[1]) * 8.0
        qb, kb = q.to(torch.bfloat16), k.to(torch.bfloat16)
        out = torch.empty(n, nq * hd, dtype=torch.bfloat16, device=DEV)
        K.attn_prefill_tc(out, qb.to(DEV), kb.to(DEV), v.to(DEV), starts, 1, n, nq, nkv, hd, 1.0, 0.0, window)
        ref = plain.attention(qb.double().reshape(n, nq, hd), kb.double().reshape(n, nkv, hd),
                              v.double().reshape(n, nkv, hd), 1.0, 0.0, window or None)
        close(out, ref, torch.bfloat16, scale=max(1.0, float(ref.abs().max())))
        visible = window == 0 or (row - far) < window
        near = (out[row].double().cpu().reshape(nq, hd) - v[far].double()).abs().max()
        assert (near < 0.05) == visible, (window, far, float(near))
    # keys whose score with every query grows by 3 per 64 positions: the maximum moves again and again
    u = torch.randn(hd)
    u = u / u.norm()
    qg = (u * 4.0).repeat(n, nq)
    kg = torch.stack([u * (0.75 * (j // 64)) for j in range(n)]) + torch.randn(n, hd) * 0.01
    qb, kb = qg.to(torch.bfloat16), kg.to(torch.bfloat16)
    out = torch.empty(n, nq * hd, dtype=torch.bfloat16, device=DEV)
    K.attn_prefill_tc(out, qb.to(DEV), kb.to(DEV), v.to(DEV), starts, 1, n, nq, nkv, hd, 1.0, 0.0, 0)
    K.check_device_errors(DEV)
    ref = plain.attention(qb.double().reshape(n, nq, hd), kb.double().reshape(n, nkv, hd),
                          v.double().reshape(n, nkv, hd), 1.0, 0.0, None)
    close(out, ref, torch.bfloat16, scale=max(1.0, float(ref.abs().max())))


def test_a_wait_that_runs_out_sets_the_error_word_and_the_library_goes_on(K):
    """The give-up path of the bounded waits for real: a barrier nobody arrives on, a limit of 2 ms.  The
    kernel returns by itself, the error word is set and is reported once, and the next product is right."""
    import time
    K.check_device_errors(DEV)                         # (clean before)
    t0 = time.perf_counter()
    waited_ms = K.selftest_wait_runs_out(DEV, limit_ms=2.0)
    torch.cuda.synchronize()
    host_ms = (time.perf_counter() - t0) * 1e3
    assert 2.0 <= waited_ms < 20.0, waited_ms          # it waited for its limit and not much longer
    assert host_ms < 2000.0
    assert int(K.error_word(DEV).item()) == 1
    with pytest.raises(K.KernelError, match="gave up waiting"):
        K.check_device_errors(DEV)
    K.check_device_errors(DEV)                         # reported once, then clear
    x = torch.randn(8, 256).to(torch.bfloat16)
    w = (torch.randn(384, 256) * 0.05).to(torch.bfloat16)
    out = torch.empty(8, 384, dtype=torch.float32, device=DEV)
    K.gemm_tc(out, x.to(DEV), w.to(DEV))
    K.check_device_errors(DEV)
    close(out, x.double() @ w.double().T, torch.float32)
    with pytest.raises(K.KernelError, match="100 ms"):
        K.selftest_wait_runs_out(DEV, limit_ms=5000.0)


def test_attention_decode_random_shapes_agree_with_the_plain_kernel(K):
    """Fifty random steps (head sizes, groups of up to 20 heads, 1 to 200 sequences of every mix of lengths, windows,
    rows without a slot, any room for partial results, with and without the step's plan): the split kernel's cut
    must cover every page of every sequence once, whatever the shapes; the plain kernel walks the keys one by one."""
    import random
    rng = random.Random(20)
    ran = 0
    while ran < 50:
        hd = rng.choice([64, 128, 256])
        nkv = rng.choice([1, 2, 4, 8])
        nq = nkv * rng.choice([1, 2, 3, 8, 17, 20])
        if nq * hd > 8192:
            continue
        B = rng.choice([1, 2, 3, 7, 8, 31, 32, 33, 64, 65, 100, 150, 200])
        kind = rng.choice(["short", "mixed", "long1", "equal", "tiny"])
        if kind == "short":
            lens = [rng.randint(1, 200) for _ in range(B)]
        elif kind == "mixed":
            lens = [rng.randint(1, 1500) for _ in range(B)]
        elif kind == "long1":
            lens = [rng.randint(1, 100) for _ in range(B)]
            lens[rng.randrange(B)] = rng.randint(2000, 5000)
        elif kind == "equal":
            lens = [rng.choice([64, 65, 128, 700, 1024])] * B
        else:
            lens = [rng.randint(1, 3) for _ in range(B)]
        window = rng.choice([0, 0, 64, 100, 257, 1024])
        ring = ((window + PAGE - 1) // PAGE) * PAGE if window else 0
        per_seq = max(((min(n, ring) if ring else n) + PAGE - 1) // PAGE for n in lens)
        n_pages = B * per_seq + 1
        if n_pages * nkv * PAGE * hd * 4 > 2e9:
            continue
        ran += 1
        g = torch.Generator().manual_seed(ran)
        table = (torch.randperm(n_pages - 1, generator=g)[: B * per_seq].reshape(B, per_seq) + 1).to(torch.int32).to(DEV)
        kc = (torch.randn(n_pages, nkv, PAGE, hd, device=DEV) * 0.3).bfloat16()
        vc = torch.randn(n_pages, nkv, PAGE, hd, device=DEV).bfloat16()
        slots = torch.tensor([-1 if rng.random() < 0.15 else b for b in range(B)], dtype=torch.int32, device=DEV)
        lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
        q = torch.randn(B, nq * hd, device=DEV).bfloat16()
        scale, cap = 1.0 / math.sqrt(hd), rng.choice([0.0, 30.0])
        ref = torch.empty(B, nq * hd, dtype=torch.bfloat16, device=DEV)
        K.attn_decode_plain(ref, q, kc, vc, table, slots, lens_t, nq, nkv, hd, scale, cap, window, ring)
        for room in (K.attn_decode_max_splits(B, nkv, max(lens), window, nq=nq), rng.choice([1, 2, 3, 4, 7])):
            for use_plan in (False, True):
                out = torch.full((B, nq * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
                plan = K.attn_decode_plan(table, slots, lens_t, nq, nkv, window, ring, room) if use_plan else None
                K.attn_decode_split(out, q, kc, vc, table, slots, lens_t, nq, nkv, hd, scale, cap, window, ring, room,
                                    plan=plan)
                K.check_device_errors(DEV)
                off = float((out.float() - ref.float()).abs().max())
                assert off <= 1.2e-2 * max(1.0, float(ref.float().abs().max())), \
                    dict(hd=hd, nq=nq, nkv=nkv, B=B, kind=kind, window=window, room=room, plan=use_plan, off=off)


def test_attention_decode_refuses_a_plan_of_another_launch(K):
    """A plan made for other room than the call's is not followed: the error word is raised, nothing is read
    through it."""
    dtype, hd, nq, nkv = torch.bfloat16, 128, 4, 2
    lens = [100, 300]
    table = torch.arange(10, dtype=torch.int32).reshape(2, 5).to(DEV)
    kc = torch.zeros(10, nkv, PAGE, hd, dtype=dtype, device=DEV)
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
    q = torch.zeros(2, nq * hd, dtype=dtype, device=DEV)
    out = torch.zeros_like(q)
    plan = K.attn_decode_plan(table, slots, lens_t, nq, nkv, 0, 0, 7)
    K.attn_decode_split(out, q, kc, kc, table, slots, lens_t, nq, nkv, hd, 1.0, 0.0, 0, 0, 9, plan=plan)
    torch.cuda.synchronize()
    with pytest.raises(K.KernelError):
        K.check_device_errors(DEV)
    K.check_device_errors(DEV)   # (the word is cleared by the check)


@pytest.mark.parametrize("hd", [256, 80, 128])
def test_rope_with_the_table_of_the_step_gives_the_same_bits(K, hd):
    """Many bfloat16 rows: the kernel takes cosines and sines from the step's table, which holds the same 32-bit
    values that it works out itself without one; the rows and the cache come out bit for bit the same, and right."""
    dtype, nq, nkv, theta = torch.bfloat16, 4, 2, 10000.0
    lens = [150, 40]
    T = sum(lens)
    torch.manual_seed(hd)
    qkv = torch.randn(T, (nq + 2 * nkv) * hd).to(dtype)
    pos = torch.tensor(list(range(150)) + list(range(40)), dtype=torch.int32, device=DEV)
    seq = torch.tensor([0] * 150 + [1] * 40, dtype=torch.int32, device=DEV)
    inv = (torch.tensor(theta, dtype=torch.float64) ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float().to(DEV)
    table = torch.tensor([[4, 2, 0], [1, -1, -1]], dtype=torch.int32, device=DEV)
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEV)
    outs = []
    for with_table in (False, True):
        d = qkv.to(DEV)
        kc = torch.zeros(5, nkv, PAGE, hd, dtype=dtype, device=DEV)
        vc = torch.zeros_like(kc)
        tb = K.rope_table(pos, inv) if with_table else None
        K.rope_cache_write(d, pos, inv, nq, nkv, hd, hd, "half", seq_of_token=seq, slots=slots, len_after=lens_t,
                           kcache=kc, vcache=vc, page_table=table, ring_rows=0, table=tb)
        outs.append((d, kc, vc))
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    x = qkv.double().reshape(T, nq + 2 * nkv, hd)
    want = torch.cat([plain.rope(x[:, : nq + nkv], pos.tolist(), theta), x[:, nq + nkv:]], 1)
    close(outs[1][0].reshape(T, -1, hd), want, dtype)
    assert torch.equal(outs[1][1][4, 0, 5].cpu(), outs[1][0].cpu().reshape(T, -1, hd)[5, nq])     # k of token 5, kv head 0
    with pytest.raises(K.KernelError, match="table"):
        K.rope_cache_write(qkv.to(DEV), pos, inv, nq, nkv, hd, hd, "half", table=K.rope_table(pos[:10], inv))
