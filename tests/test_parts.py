"""Each part alone against the plain implementation; parts of other kinds
than the model's built and run; a layer run twice and a layer that reads
another layer's cache."""
import copy
import math

import pytest
import torch

import plain_gemma2 as plain
import replay
from tiny import CONFIGS, TINY_B, make_folder
from tolerances import FP32_VS_PLAIN, rel_err

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _ctx(dtype=torch.float32):
    from airframe_b200.parts import BuildContext
    return BuildContext(dtype, DEV)


def _batch(lens_before, tokens_per_seq, slots=None):
    from airframe_b200.engine import StepEntry, build_batch
    entries = [StepEntry(s if slots is None else slots[i], [0] * n, []) for i, (s, n) in
               enumerate(zip(range(len(tokens_per_seq)), tokens_per_seq))]
    return build_batch(entries, lens_before, DEV)


def test_norm_part_alone():
    from airframe_b200.config import PartSpec
    from airframe_b200.parts import build_part
    H = 200
    n = build_part("norm", PartSpec("rms_norm", {"weight": "w", "size": H, "eps": 1e-5, "weight_offset": 1.0}), _ctx())
    assert [(d.name, d.shape, d.kind) for d in n.weight_decls()] == [("w", (H,), "norm")]
    w = torch.randn(H) * 0.1
    n.load({"w": w.to(DEV).to(torch.bfloat16)})                     # stored in 16 bits: widened exactly
    x = torch.randn(6, H)
    got = n.forward(x.to(DEV), torch.float32)
    assert rel_err(got, plain.rms_norm(x.double(), w.to(torch.bfloat16).double(), 1e-5)) < 1e-5
    a = torch.randn(6, H)
    xd = x.to(DEV)
    assert n.add_normed(xd, a.to(DEV)) is None
    assert rel_err(xd, x.double() + plain.rms_norm(a.double(), w.to(torch.bfloat16).double(), 1e-5)) < 1e-5


def test_gated_mlp_part_alone_with_both_activations():
    from airframe_b200.config import ConfigError, PartSpec
    from airframe_b200.parts import build_part
    H, I = 72, 200
    ws = {"g": torch.randn(I, H) * 0.1, "u": torch.randn(I, H) * 0.1, "d": torch.randn(H, I) * 0.1}
    x = torch.randn(5, H)
    for act, fn in (("gelu_tanh", plain.gelu_tanh), ("silu", lambda g: g * torch.sigmoid(g))):
        p = {"hidden_size": H, "intermediate_size": I, "activation": act, "gate_weight": "g", "up_weight": "u",
             "down_weight": "d"}
        m = build_part("feed_forward", PartSpec("gated_mlp", p), _ctx())
        m.load({k: v.to(DEV) for k, v in ws.items()})
        got = m.forward(x.to(DEV), None)
        xd, g, u, d = x.double(), ws["g"].double(), ws["u"].double(), ws["d"].double()
        assert rel_err(got, (fn(xd @ g.T) * (xd @ u.T)) @ d.T) < 1e-5
    with pytest.raises(ConfigError, match="unknown activation"):
        build_part("feed_forward", PartSpec("gated_mlp", dict(p, activation="relu")), _ctx())
    with pytest.raises(ConfigError, match="no feed_forward part of kind 'experts'"):
        build_part("feed_forward", PartSpec("experts", {}), _ctx())


def test_attention_part_alone_prefill_then_decode():
    """The mixer with a cache of its own: two sequences, prompts then three
    single tokens, against the plain attention on the whole sequences."""
    from airframe_b200.cache import SequenceCache
    from airframe_b200.config import PartSpec
    from airframe_b200.engine import StepEntry, build_batch
    from airframe_b200.parts import build_part
    H, nq, nkv, hd, W = 80, 5, 1, 32, 9
    p = {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd, "scale": 0.2, "softcap": 10.0,
         "window": W, "position": PartSpec("rope", {"theta": 777.0, "rotary_dim": hd, "pairing": "half"}),
         "q_weight": "q", "k_weight": "k", "v_weight": "v", "o_weight": "o"}
    att = build_part("mixer", PartSpec("attention", p), _ctx())
    ws = {"q": torch.randn(nq * hd, H) * 0.1, "k": torch.randn(nkv * hd, H) * 0.1,
          "v": torch.randn(nkv * hd, H) * 0.1, "o": torch.randn(H, nq * hd) * 0.1}
    att.load({k: v.to(DEV) for k, v in ws.items()})
    cache = SequenceCache([(att.kv_need(), att.state_need(), None)], 64 * 4, 128, torch.float32, DEV)
    lens = [13, 4]
    xs = [torch.randn(n + 3, H) for n in lens]
    slots = [cache.take_slot(), cache.take_slot()]

    def want(x):
        T = x.shape[0]
        xd = x.double()
        q = plain.rope((xd @ ws["q"].double().T).reshape(T, nq, hd), range(T), 777.0)
        k = plain.rope((xd @ ws["k"].double().T).reshape(T, nkv, hd), range(T), 777.0)
        v = (xd @ ws["v"].double().T).reshape(T, nkv, hd)
        return plain.attention(q, k, v, 0.2, 10.0, W) @ ws["o"].double().T

    refs = [want(x) for x in xs]
    cache.reserve({s: n for s, n in zip(slots, lens)})
    cache.flush()
    b = build_batch([StepEntry(s, [0] * n, []) for s, n in zip(slots, lens)], [0, 0], DEV)
    got = att.forward(torch.cat([x[:n] for x, n in zip(xs, lens)]).to(DEV), b, cache.views[0])
    cache.commit({s: n for s, n in zip(slots, lens)})
    assert rel_err(got[:13], refs[0][:13]) < 1e-5 and rel_err(got[13:], refs[1][:4]) < 1e-5
    for step in range(3):
        now = [n + step for n in lens]
        cache.reserve({s: n + 1 for s, n in zip(slots, now)})
        cache.flush()
        b = build_batch([StepEntry(s, [0], []) for s in slots], now, DEV)
        got = att.forward(torch.stack([x[n] for x, n in zip(xs, now)]).to(DEV), b, cache.views[0])
        cache.commit({s: n + 1 for s, n in zip(slots, now)})
        assert rel_err(got[0], refs[0][now[0]]) < 1e-5 and rel_err(got[1], refs[1][now[1]]) < 1e-5


def test_prenorm_block_with_silu_and_adjacent_rope_builds_and_matches():
    """Other kinds than Gemma-2's in every slot, assembled by the same builder:
    a pre-norm block, plain weights (offset 0), SiLU, adjacent rotary pairs on
    half of the head, no softcaps, untied head."""
    from airframe_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from airframe_b200.engine import Engine, Model, StepEntry
    from airframe_b200.weights import RandomSource, load_weights
    H, V, nq, nkv, hd, I = 48, 90, 3, 3, 16, 100

    def norm(name):
        return PartSpec("rms_norm", {"weight": name, "size": H, "eps": 1e-5, "weight_offset": 0.0})

    layers = []
    for i in range(2):
        p = f"l{i}."
        mixer = PartSpec("attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd,
                                       "scale": hd ** -0.5, "softcap": 0.0, "window": None,
                                       "position": PartSpec("rope", {"theta": 100.0, "rotary_dim": 8, "pairing": "adjacent"}),
                                       "q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "o_weight": p + "o"})
        ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
                                     "gate_weight": p + "g", "up_weight": p + "u", "down_weight": p + "d"})
        layers.append(LayerSpec(p, PartSpec("prenorm"), mixer, ffn,
                                {"pre_mixer": norm(p + "n1"), "pre_feed_forward": norm(p + "n2")}))
    spec = ModelSpec("toy", H, V, 64, PartSpec("token_embedding", {"weight": "emb", "vocab_size": V, "hidden_size": H, "scale": 1.0}),
                     layers, [ScheduleEntry(0), ScheduleEntry(1)], norm("nf"),
                     PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "softcap": 0.0, "weight": "head"}))
    model = Model(spec, torch.float32, DEV)
    decls = model.weight_decls()
    assert {d.name for d in decls} >= {"emb", "head", "l0.q", "l1.n2", "nf"}
    wts = load_weights(RandomSource(decls, 5, torch.float32), decls, torch.float32, DEV)
    model.load(wts)
    eng = Engine(model, 64 * 2)
    ids = replay.random_ids(V, 20, 1)
    s = eng.take_slot()
    got = torch.cat([eng.step([StepEntry(s, ids[:12], list(range(12)))])] +
                    [eng.step([StepEntry(s, [t], [0])]) for t in ids[12:]])
    w = {k: v.double().cpu() for k, v in wts.items()}

    def rms(x, wt):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * wt

    def rope_adj(x):                                  # adjacent pairs on the first 8 of 16
        T = x.shape[0]
        part = torch.cat([x[..., 0:8:2], x[..., 1:8:2]], -1)
        r = plain.rope(part, range(T), 100.0)
        out = x.clone()
        out[..., 0:8:2], out[..., 1:8:2] = r[..., :4], r[..., 4:]
        return out

    x = w["emb"][ids]
    T = len(ids)
    for i in range(2):
        p = f"l{i}."
        h = rms(x, w[p + "n1"])
        q, k = rope_adj((h @ w[p + "q"].T).reshape(T, nq, hd)), rope_adj((h @ w[p + "k"].T).reshape(T, nkv, hd))
        v = (h @ w[p + "v"].T).reshape(T, nkv, hd)
        x = x + plain.attention(q, k, v, hd ** -0.5, 0.0, None) @ w[p + "o"].T
        h = rms(x, w[p + "n2"])
        g = h @ w[p + "g"].T
        x = x + (g * torch.sigmoid(g) * (h @ w[p + "u"].T)) @ w[p + "d"].T
    ref = rms(x, w["nf"]) @ w["head"].T
    assert rel_err(got, ref) < FP32_VS_PLAIN


def test_a_layer_run_twice_and_a_layer_reading_anothers_cache(tmp_path):
    """The schedule is data: [0, 1, 0 again, 2 reading the keys and values of
    the second run].  Checked against the plain parts put together the same way,
    whole and with the last tokens one by one (prompt longer than the ring)."""
    from airframe_b200.config import ScheduleEntry, config_from_dict
    from airframe_b200.engine import Engine, Model, StepEntry
    from airframe_b200.weights import SafetensorsFolder, load_weights
    cfgd = dict(TINY_B, layer_types=["sliding_attention", "full_attention", "full_attention"])
    folder = make_folder(cfgd, seed=8, store_dtype="float32", root=tmp_path)
    cfg, w = plain.read_model_folder(folder)
    spec = config_from_dict(cfgd).model_spec()
    spec.schedule = [ScheduleEntry(0), ScheduleEntry(1), ScheduleEntry(0), ScheduleEntry(2, cache_from=1)]
    model = Model(spec, torch.float32, DEV)
    model.load(load_weights(SafetensorsFolder(folder), model.weight_decls(), torch.float32, DEV))
    eng = Engine(model, 64 * 4)
    assert len(eng.cache.groups) == 2 and eng.cache.views[3].cache_id == 1 and not eng.cache.views[3].writes
    ids = replay.random_ids(cfg["vocab_size"], 90, 2)

    # the plain parts in the same order; the last run attends with its own queries to run 1's keys and values
    T = len(ids)
    pos = list(range(T))
    x = plain.embed(ids, w["model.embed_tokens.weight"], cfg["hidden_size"])
    x = plain.block(x, pos, 0, cfg, w)
    nq, nkv, hd, eps = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"], cfg["rms_norm_eps"]
    n1 = plain.rms_norm(x, w["model.layers.1.input_layernorm.weight"], eps)
    k1 = plain.rope((n1 @ w["model.layers.1.self_attn.k_proj.weight"].T).reshape(T, nkv, hd), pos, cfg["rope_theta"])
    v1 = (n1 @ w["model.layers.1.self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
    c = dict(cfg)
    x = plain.block(x, pos, 1, dict(cfg, sliding_window=10 ** 9), w)      # layer 1 is global here
    x = plain.block(x, pos, 0, cfg, w)                                     # layer 0 again (local)
    p = "model.layers.2."
    n = plain.rms_norm(x, w[p + "input_layernorm.weight"], eps)
    q = plain.rope((n @ w[p + "self_attn.q_proj.weight"].T).reshape(T, nq, hd), pos, cfg["rope_theta"])
    a = plain.attention(q, k1, v1, cfg["query_pre_attn_scalar"] ** -0.5, cfg["attn_logit_softcapping"], None)
    x = x + plain.rms_norm(a @ w[p + "self_attn.o_proj.weight"].T, w[p + "post_attention_layernorm.weight"], eps)
    n2 = plain.rms_norm(x, w[p + "pre_feedforward_layernorm.weight"], eps)
    f = plain.geglu_mlp(n2, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    x = x + plain.rms_norm(f, w[p + "post_feedforward_layernorm.weight"], eps)
    ref = plain.lm_head(x, cfg, w)

    s = eng.take_slot()
    whole = eng.step([StepEntry(s, ids, list(range(T)))])
    eng.free_slot(s)
    assert rel_err(whole, ref) < FP32_VS_PLAIN
    s = eng.take_slot()
    tail = torch.cat([eng.step([StepEntry(s, ids[:70], list(range(70)))])] +
                     [eng.step([StepEntry(s, [t], [0])]) for t in ids[70:]])
    assert rel_err(tail, ref) < FP32_VS_PLAIN
