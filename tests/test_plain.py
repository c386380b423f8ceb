"""The plain implementation checked against hand-made cases, in the manner of
the reference's unit tests of its CPU operations (identities, visibility,
first-max tie rule).  No GPU."""
import math

import numpy as np
import pytest
import torch

import plain_gemma2 as plain
from tiny import TINY_A, TINY_B, make_folder


@pytest.fixture(scope="module")
def model_a(tmp_path_factory):
    return plain.read_model_folder(make_folder(TINY_A, seed=2, root=tmp_path_factory.mktemp("a")))


def test_rope_identity_at_position_zero_and_norm_kept():
    x = torch.randn(3, 2, 8, dtype=torch.float64)
    assert torch.allclose(plain.rope(x, [0, 0, 0], 10000.0), x)            # src/ops/dispatch.rs:417-429
    y = plain.rope(x, [5, 9, 300], 10000.0)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    assert not torch.allclose(y, x)


def test_rope_scores_depend_on_distance_only():
    q = torch.randn(1, 1, 16, dtype=torch.float64)
    k = torch.randn(1, 1, 16, dtype=torch.float64)
    def score(m, n):
        return (plain.rope(q, [m], 1e4) * plain.rope(k, [n], 1e4)).sum()
    assert score(7, 3) == pytest.approx(score(104, 100), abs=1e-9)          # sh_layer_v1.wgsl:706-725
    assert abs(score(7, 3) - score(7, 4)) > 1e-6
    # pairs are (i, i + hd/2): a vector with only element 0 and hd/2 set stays in that plane
    e = torch.zeros(1, 1, 16, dtype=torch.float64)
    e[0, 0, 0] = 1.0
    r = plain.rope(e, [1], 1e4)[0, 0]
    assert r[0] == pytest.approx(math.cos(1.0)) and r[8] == pytest.approx(math.sin(1.0))
    assert r[1] == 0 and r[9] == 0


def test_rms_norm_uses_one_plus_w():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = plain.rms_norm(x, torch.tensor([0.0, 1.0], dtype=torch.float64), 0.0)
    assert torch.allclose(y, torch.tensor([[3.0, 8.0]], dtype=torch.float64) / math.sqrt(12.5))


def test_visibility_window_edges():
    m = plain.visibility(6, 3)
    assert m[5].tolist() == [False, False, False, True, True, True]         # i - j < 3
    assert m[1].tolist() == [True, True, False, False, False, False]
    assert plain.visibility(4, None).tolist() == torch.tril(torch.ones(4, 4)).bool().tolist()


def test_attention_weights_sum_to_one_and_heads_map_to_groups():
    T, nq, nkv, hd = 5, 4, 2, 8
    q, k = torch.randn(T, nq, hd, dtype=torch.float64), torch.randn(T, nkv, hd, dtype=torch.float64)
    v = torch.ones(T, nkv, hd, dtype=torch.float64)
    v[:, 1] = 2.0
    out = plain.attention(q, k, v, 0.3, 50.0, None).reshape(T, nq, hd)
    assert torch.allclose(out[:, :2], torch.ones(T, 2, hd, dtype=torch.float64))      # heads 0,1 -> group 0
    assert torch.allclose(out[:, 2:], 2 * torch.ones(T, 2, hd, dtype=torch.float64))  # heads 2,3 -> group 1


def test_softcap_bounds_and_is_identity_when_off():
    s = torch.tensor([-1e4, -1.0, 0.0, 2.0, 1e4], dtype=torch.float64)
    c = plain.softcap(s, 30.0)
    assert c.abs().max() <= 30.0 and c[2] == 0 and c[3] == pytest.approx(30 * math.tanh(2 / 30))
    assert plain.softcap(s, None) is s and plain.softcap(s, 0.0) is s


def test_gelu_tanh_values():
    g = torch.tensor([0.0, 1.0, -1.0], dtype=torch.float64)
    y = plain.gelu_tanh(g)
    assert y[0] == 0 and y[1] == pytest.approx(0.841192, abs=1e-6) and y[2] == pytest.approx(-0.158808, abs=1e-6)


def test_logits_are_causal(model_a):
    cfg, w = model_a
    ids = [5, 9, 200, 31, 77, 1, 2, 3, 4, 5, 6, 7]
    a = plain.logits(cfg, w, ids)
    b = plain.logits(cfg, w, ids[:6] + [100, 101, 102, 103, 104, 105])
    assert torch.allclose(a[:6], b[:6], atol=1e-12) and not torch.allclose(a[6:], b[6:])
    assert a.abs().max() <= cfg["final_logit_softcapping"]


def test_local_layer_sees_only_its_window(model_a):
    cfg, w = model_a                      # layer 0 is local with a window of 8
    ids = list(range(20, 40))
    other = [99] * 5 + ids[5:]
    a = plain.hidden_states(cfg, w, ids, upto_layer=1)
    b = plain.hidden_states(cfg, w, other, upto_layer=1)
    assert torch.allclose(a[12:], b[12:], atol=1e-12)        # position 12 sees 5..12
    assert not torch.allclose(a[11], b[11], atol=1e-9)       # position 11 still sees 4
    full = plain.hidden_states(cfg, w, ids)                  # layer 1 is global: everything matters
    assert not torch.allclose(full[19], plain.hidden_states(cfg, w, other)[19], atol=1e-9)


def test_greedy_takes_the_first_maximum_over_finite_values():
    assert plain.greedy([0.1, 0.9, 0.9, 0.2]) == 1                           # src/runtime/sampling.rs:71-77
    assert plain.greedy([np.nan, np.inf, 3.0, -np.inf]) == 2
    assert plain.greedy([np.nan, np.nan]) == 0


def test_repetition_penalty_once_per_occurrence():
    row = plain.apply_repetition_penalty([2.0, -2.0, 1.0], [0, 1, 0], 2.0)
    assert row.tolist() == [0.5, -4.0, 1.0]


def test_sample_token_walks_the_nucleus():
    row = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float32))
    # top_p 0.9: nucleus {0, 1, 2} (0.5 + 0.3 < 0.9 <= 0.95), mass 0.95
    assert plain.sample_token(row, 1.0, 0.9, 1.0, [], 0.0) == 0
    assert plain.sample_token(row, 1.0, 0.9, 1.0, [], 0.5) == 0             # r = 0.475 <= 0.5
    assert plain.sample_token(row, 1.0, 0.9, 1.0, [], 0.6) == 1             # r = 0.57
    assert plain.sample_token(row, 1.0, 0.9, 1.0, [], 0.99) == 2
    assert plain.sample_token(row, 1.0, 0.4, 1.0, [], 0.99) == 0            # nucleus {0}
    assert plain.sample_token(row, 0.0, 0.9, 1.0, [], 0.99) == 0            # greedy
    assert plain.sample_token(row, 0.0, 0.9, 100.0, [0], 0.99) == 1         # penalty first


def test_xorshift_is_deterministic_and_in_range():
    a, b = plain.XorShift64Star(42), plain.XorShift64Star(42)
    xs = [a.next_f32() for _ in range(100)]
    assert xs == [b.next_f32() for _ in range(100)]
    assert all(0.0 <= x < 1.0 for x in xs) and len(set(xs)) > 90
    # first value by hand: state 43
    s = 43
    s ^= s >> 12
    s ^= (s << 25) & (2 ** 64 - 1)
    s ^= s >> 27
    assert xs[0] == np.float32(((s * 0x2545F4914F6CDD1D) & (2 ** 64 - 1)) >> 40) / np.float32(16777216.0)
    from airframe_b200.sampling import XorShift64Star
    c = XorShift64Star(42)
    assert [c.next_f32() for _ in range(100)] == [float(x) for x in xs]


def test_score_scale_is_query_pre_attn_scalar_not_head_dim(model_a):
    """Gemma-2's own: scores are scaled by query_pre_attn_scalar^-0.5 (27B: 144 with head_dim 128)."""
    cfg, w = model_a
    ids = [5, 17, 3, 200, 9, 41]
    base = plain.logits(cfg, w, ids)
    other = plain.logits(dict(cfg, query_pre_attn_scalar=cfg["query_pre_attn_scalar"] * 4), w, ids)
    assert not torch.allclose(base, other)
    # one layer by hand: the block's attention equals attention() called with that scale
    x = plain.embed(ids, w["model.embed_tokens.weight"], cfg["hidden_size"])
    h = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    pos = list(range(len(ids)))
    q = plain.rope((h @ w["model.layers.1.self_attn.q_proj.weight"].T).reshape(-1, nq, hd), pos, cfg["rope_theta"])
    k = plain.rope((h @ w["model.layers.1.self_attn.k_proj.weight"].T).reshape(-1, nkv, hd), pos, cfg["rope_theta"])
    v = (h @ w["model.layers.1.self_attn.v_proj.weight"].T).reshape(-1, nkv, hd)
    ctx = plain.attention(q, k, v, cfg["query_pre_attn_scalar"] ** -0.5, cfg["attn_logit_softcapping"], None)
    a = ctx @ w["model.layers.1.self_attn.o_proj.weight"].T
    want = x + plain.rms_norm(a, w["model.layers.1.post_attention_layernorm.weight"], cfg["rms_norm_eps"])
    # layer 1 is a global layer (odd layers see all keys): the block's first half gives the same
    got = plain.block(x, pos, 1, cfg, w)
    n2 = plain.rms_norm(want, w["model.layers.1.pre_feedforward_layernorm.weight"], cfg["rms_norm_eps"])
    f = plain.geglu_mlp(n2, w["model.layers.1.mlp.gate_proj.weight"], w["model.layers.1.mlp.up_proj.weight"],
                        w["model.layers.1.mlp.down_proj.weight"])
    want = want + plain.rms_norm(f, w["model.layers.1.post_feedforward_layernorm.weight"], cfg["rms_norm_eps"])
    assert torch.allclose(got, want, atol=1e-12)
