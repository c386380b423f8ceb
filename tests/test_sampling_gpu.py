"""The device sampler against the plain implementation."""
import numpy as np
import pytest
import torch

import plain_gemma2 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def K():
    from airframe_b200 import kernels
    return kernels


def _sample(K, rows, temperature, top_p, penalty, u=None, recent=None):
    logits = torch.tensor(np.asarray(rows, dtype=np.float32), device=DEV)
    R = logits.shape[0]
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    rec = nrec = None
    if recent is not None:
        rec = torch.zeros(R, 64, dtype=torch.int32)
        nrec = torch.zeros(R, dtype=torch.int32)
        for r, lst in enumerate(recent):
            rec[r, : len(lst)] = torch.tensor(lst, dtype=torch.int32)
            nrec[r] = len(lst)
        rec, nrec = rec.to(DEV), nrec.to(DEV)
    uni = torch.tensor(u, dtype=torch.float32, device=DEV) if u is not None else None
    K.sample(logits, out, temperature, top_p, penalty, uniform=uni, recent=rec, n_recent=nrec)
    return out.tolist(), logits.cpu().numpy()


@pytest.mark.parametrize("V", [7, 256, 1000, 256000])
def test_greedy_is_the_first_finite_maximum(K, V):
    rng = np.random.default_rng(V)
    rows = rng.standard_normal((5, V)).astype(np.float32)
    rows[1, [V // 3, V // 2]] = 9.0                     # a tie: the lower index wins
    rows[2, 0] = np.inf
    rows[2, V - 1] = np.nan
    rows[3, :] = np.nan
    got, _ = _sample(K, rows, 0.0, 0.95, 1.0)
    assert got == [plain.greedy(r) for r in rows]
    assert got[1] == V // 3 and got[3] == 0


def test_repetition_penalty_changes_the_winner(K):
    rows = np.array([[1.0, 3.0, 2.9, -1.0], [1.0, -0.5, -0.4, -3.0]], dtype=np.float32)
    got, changed = _sample(K, rows, 0.0, 1.0, 1.5, recent=[[1, 1], [2, 0, 2]])
    assert got == [2, 0]
    want0 = plain.apply_repetition_penalty(rows[0], [1, 1], 1.5)
    want1 = plain.apply_repetition_penalty(rows[1], [2, 0, 2], 1.5)
    assert np.allclose(changed[0], want0) and np.allclose(changed[1], want1)
    assert got == [plain.greedy(want0), plain.greedy(want1)]


def _nucleus(row, temperature, top_p):
    """The reference's nucleus (src/runtime/gpu.rs:924-948) in 64 bits: ids and probabilities."""
    z = np.asarray(row, dtype=np.float64) / temperature
    p = np.exp(z - z.max())
    p /= p.sum()
    order = np.argsort(-p, kind="stable")
    cum = np.cumsum(p[order])
    cutoff = int(np.searchsorted(cum, top_p - 1e-12) + 1)
    return order[:cutoff], p


@pytest.mark.parametrize("V,temperature,top_p", [(50, 0.8, 0.95), (1000, 1.0, 0.5), (1000, 0.3, 0.9),
                                                 (256000, 0.8, 0.95), (4000, 1.5, 1.0)])
def test_draw_lands_where_the_uniform_number_points(K, V, temperature, top_p):
    """The token drawn with u is the one whose interval of the nucleus's
    cumulative mass, in index order, holds u."""
    rng = np.random.default_rng(V + int(100 * top_p))
    R = 16
    rows = (rng.standard_normal((R, V)) * 2).astype(np.float32)
    u = rng.random(R).astype(np.float32)
    u[0], u[1] = 0.0, 0.99999994
    got, _ = _sample(K, rows, temperature, top_p, 1.0, u=u)
    for r in range(R):
        ids, p = _nucleus(rows[r], temperature, top_p)
        inside = np.zeros(V, dtype=bool)
        inside[ids] = True
        assert inside[got[r]], (r, got[r])
        w = np.where(inside, p, 0.0)
        cum = np.cumsum(w)
        mass = cum[-1]
        lo, hi = (cum[got[r]] - w[got[r]]) / mass, cum[got[r]] / mass
        assert lo - 1e-4 <= u[r] <= hi + 1e-4, (r, lo, float(u[r]), hi)


def test_top_p_keeps_the_tail_out_and_frequencies_follow_the_probabilities(K):
    probs = np.array([0.4, 0.3, 0.2, 0.06, 0.04])
    row = np.log(probs).astype(np.float32)
    n = 4000
    rows = np.tile(row, (n, 1))
    u = np.random.default_rng(0).random(n).astype(np.float32)
    got, _ = _sample(K, rows, 1.0, 0.9, 1.0, u=u)
    counts = np.bincount(got, minlength=5) / n
    assert counts[3] == 0 and counts[4] == 0            # 0.4 + 0.3 + 0.2 reaches 0.9
    assert np.allclose(counts[:3], probs[:3] / 0.9, atol=0.03)
    got, _ = _sample(K, rows, 1.0, 1.0, 1.0, u=u)
    assert np.allclose(np.bincount(got, minlength=5) / n, probs, atol=0.03)


def test_ties_at_the_cutoff_enter_lowest_index_first(K):
    row = np.log(np.array([0.25, 0.25, 0.25, 0.25])).astype(np.float32)
    # top_p 0.5 needs two of the four equal tokens: 0 and 1
    rows = np.tile(row, (64, 1))
    u = np.linspace(0, 0.999, 64).astype(np.float32)
    got, _ = _sample(K, rows, 1.0, 0.5, 1.0, u=u)
    assert set(got) == {0, 1} and got == sorted(got)


def test_a_row_does_not_depend_on_its_batch(K):
    rng = np.random.default_rng(9)
    rows = rng.standard_normal((8, 5000)).astype(np.float32)
    u = rng.random(8).astype(np.float32)
    together, _ = _sample(K, rows, 0.8, 0.95, 1.1, u=u, recent=[[1, 2, 3]] * 8)
    alone = [_sample(K, rows[i:i + 1], 0.8, 0.95, 1.1, u=u[i:i + 1], recent=[[1, 2, 3]])[0][0] for i in range(8)]
    assert together == alone


def test_the_sampler_reports_a_kernel_that_gave_up_waiting(K):
    """Kernels with bounded waits set a device word when a wait runs out; the word travels to the host
    with the sampled tokens, and the step fails instead of returning tokens made from garbage.  (The
    word is set by hand here: no kernel is made to wait.)"""
    from airframe_b200.sampling import Sampler, SamplingParams
    sampler = Sampler(16, DEV)
    params = SamplingParams(temperature=0.0, repetition_penalty=1.0)
    logits = torch.zeros(2, 16, device=DEV)
    logits[:, 3] = 1.0
    states = [sampler.new_state(params, i) for i in range(2)]
    assert sampler.sample(logits, states, params) == [3, 3]
    K.error_word(DEV).fill_(1)
    with pytest.raises(K.KernelError, match="gave up waiting"):
        sampler.sample(logits, states, params)
    assert sampler.sample(logits, states, params) == [3, 3]          # the word was cleared


@pytest.mark.parametrize("R,V,H,cap", [(1, 1000, 64, 30.0), (8, 256000, 264, 30.0), (5, 777 * 8, 520, 0.0), (40, 5000, 128, 2.0),
                                       (130, 3000, 64, 0.0), (300, 1300, 72, 15.0)])
def test_head_with_the_arg_max_in_its_epilogue(R, V, H, cap):
    """The greedy token of every row without logits in memory: the same token as the arg-max of the logits
    the product writes (finite values, lowest id among equals), also where the cap makes many values equal."""
    from airframe_b200 import kernels as K
    g = torch.Generator().manual_seed(R * V + H)
    y = torch.randn(R, H, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(V, H, generator=g) * (3.0 if cap == 2.0 else 0.3)).to(torch.bfloat16)
    w[V // 2] = w[7]                                      # two equal rows: the lower id wins
    w = w.to(DEV)
    logits = torch.empty(R, V, dtype=torch.float32, device=DEV)
    K.gemm_tc(logits, y, w, cap=cap)
    want = []
    for r in range(R):
        row = logits[r]
        best = row[torch.isfinite(row)].max()
        want.append(int((row == best).nonzero()[0]))
    keys = torch.zeros(max(R, 4) * K.argmax_key_stride(), dtype=torch.int64, device=DEV)
    for attempt in range(2):                              # twice: the keys come back to zero
        tokens = torch.full((R,), -5, dtype=torch.int32, device=DEV)
        K.gemm_tc_argmax(tokens, y, w, cap, keys)
        K.check_device_errors(DEV)
        assert tokens.tolist() == want
        assert int(keys.abs().sum()) == 0
    if cap == 2.0:
        sat = (logits == logits.max()).sum(-1)
        assert int(sat.max()) > 1                         # the cap did make equal values somewhere
    # and against the plain implementation's arg-max over the plain logits, where its margin is clear
    ref = plain.softcap(y.double().cpu() @ w.double().cpu().T, cap if cap > 0 else None)
    top2 = ref.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > 1e-3 * ref.abs().max()
    got = torch.tensor(want)
    assert bool((got[clear] == ref.argmax(-1)[clear]).all())
