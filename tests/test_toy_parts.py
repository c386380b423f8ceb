"""Two more parts that are no model's, defined here and registered from
outside the package: a feed-forward with routing (a router picks one of
several small experts per token) and another position encoding (a learned
vector per position added to the query and key heads).  They compute with
torch; what is under test is that the registry, the weight loader, the block,
the cache, the step function and its ways of cutting the work take them
without a change to the framework's files."""
import pytest
import torch

import plain_gemma2 as plain
import replay
from tolerances import FP32_VS_PLAIN, SPLITS, rel_err

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _register():
    from airframe_b200.parts import FeedForward, PositionEncoding, build_part, register_part
    from airframe_b200.config import PartSpec
    from airframe_b200.parts.linear import linear
    from airframe_b200.weights import WeightDecl

    @register_part("feed_forward", "toy_top1_experts")
    class Top1Experts(FeedForward):
        """y_t = W2[e_t] relu(W1[e_t] x_t), e_t = argmax_e (R x_t)_e (router in 32 bits)."""

        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.h, self.i, self.e, self.p = params["hidden_size"], params["inner_size"], params["experts"], params["prefix"]

        def weight_decls(self):
            return ([WeightDecl(self.p + "router", (self.e, self.h))] +
                    [WeightDecl(f"{self.p}e{k}.w1", (self.i, self.h)) for k in range(self.e)] +
                    [WeightDecl(f"{self.p}e{k}.w2", (self.h, self.i)) for k in range(self.e)])

        def load(self, weights):
            dt = self.ctx.compute_dtype
            self.router = weights[self.p + "router"].float()
            self.w1 = [weights[f"{self.p}e{k}.w1"].to(dt).contiguous() for k in range(self.e)]
            self.w2 = [weights[f"{self.p}e{k}.w2"].to(dt).contiguous() for k in range(self.e)]

        def forward(self, x, batch):
            choice = (x.float() @ self.router.T).argmax(-1)
            out = torch.zeros_like(x)
            for k in range(self.e):
                rows = (choice == k).nonzero().flatten()          # reads the device: this part is not graph-safe
                if rows.numel():
                    hid = torch.relu(linear(x[rows].contiguous(), self.w1[k]))
                    out[rows] = linear(hid, self.w2[k])
            return out

    @register_part("position", "toy_learned_offset")
    class LearnedOffset(PositionEncoding):
        """q_h += P[pos], k_h += P[pos] for every head; the mixer stores k and v."""

        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.name, self.n, self.hd = params["weight"], params["positions"], params["head_dim"]

        def weight_decls(self):
            return [WeightDecl(self.name, (self.n, self.hd))]

        def load(self, weights):
            self.table = weights[self.name].float()

        def encode(self, qkv, batch, nq, nkv, hd, parts=None):
            if parts is not None:
                qkv.copy_(parts.sum(0))
            add = self.table[batch.positions.long()].to(qkv.dtype)            # [T, hd]
            heads = qkv.view(qkv.shape[0], nq + 2 * nkv, hd)
            heads[:, : nq + nkv] += add[:, None, :]

    @register_part("position", "toy_distance_slopes")
    class DistanceSlopes(PositionEncoding):
        """Nothing is written into q or k: head h's scores get slope_h * (key - query), slope_h = base^-(h+1)."""
        graph_safe = True

        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.base, self.heads = float(params["base"]), int(params["heads"])
            self.slopes = None

        def load(self, weights):
            self.slopes = torch.tensor([self.base ** -(h + 1) for h in range(self.heads)], dtype=torch.float32,
                                       device=self.ctx.device)

        def score_slopes(self, nq):
            assert nq == self.heads
            return self.slopes
    return Top1Experts, LearnedOffset


def test_routed_feed_forward_and_learned_positions_step_through_the_engine():
    from airframe_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from airframe_b200.engine import Engine, Model, StepEntry
    from airframe_b200.parts import known_parts, unregister_part
    from airframe_b200.weights import RandomSource, load_weights
    _register()
    try:
        assert "toy_top1_experts" in known_parts("feed_forward") and "toy_learned_offset" in known_parts("position")
        H, V, nq, nkv, hd, I, E, P = 40, 70, 4, 2, 16, 24, 3, 96

        def norm(name):
            return PartSpec("rms_norm", {"weight": name, "size": H, "eps": 1e-6, "weight_offset": 1.0})

        layers = []
        for i in range(2):
            p = f"l{i}."
            pos = PartSpec("toy_learned_offset", {"weight": p + "pos", "positions": P, "head_dim": hd})
            mixer = PartSpec("attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd,
                                           "scale": 0.3, "softcap": 10.0, "window": 9 if i == 0 else None, "position": pos,
                                           "q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "o_weight": p + "o"})
            ffn = PartSpec("toy_top1_experts", {"hidden_size": H, "inner_size": I, "experts": E, "prefix": p})
            layers.append(LayerSpec(p, PartSpec("prenorm"), mixer, ffn,
                                    {"pre_mixer": norm(p + "n1"), "pre_feed_forward": norm(p + "n2")}))
        spec = ModelSpec("toy", H, V, P, PartSpec("token_embedding", {"weight": "emb", "vocab_size": V, "hidden_size": H,
                                                                      "scale": 1.0}),
                         layers, [ScheduleEntry(0), ScheduleEntry(1)], norm("nf"),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "softcap": 0.0, "tied_to": "emb"}))
        model = Model(spec, torch.float32, DEV)
        assert not model.graph_safe                      # the routed part reads the device: steps run eagerly
        decls = model.weight_decls()
        assert {"l0.router", "l1.e2.w2", "l0.pos"} <= {d.name for d in decls}
        wts = load_weights(RandomSource(decls, 9, torch.float32), decls, torch.float32, DEV)
        # make the router decisive, so that rounding does not flip a choice between the engine and the reference
        for i in range(2):
            wts[f"l{i}.router"] = wts[f"l{i}.router"] * 50.0
        model.load(wts)
        eng = Engine(model, 64 * 8)
        reqs = [replay.random_ids(V, n, 70 + n) for n in (33, 6, 21)]
        w = {k: v.double().cpu() for k, v in wts.items()}

        def rms(x, wt):
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * (1.0 + wt)

        def reference(ids):
            T = len(ids)
            x = w["emb"][ids]
            for i in range(2):
                p = f"l{i}."
                h = rms(x, w[p + "n1"])
                off = w[p + "pos"][:T][:, None, :]
                q = (h @ w[p + "q"].T).reshape(T, nq, hd) + off
                k = (h @ w[p + "k"].T).reshape(T, nkv, hd) + off
                v = (h @ w[p + "v"].T).reshape(T, nkv, hd)
                x = x + plain.attention(q, k, v, 0.3, 10.0, 9 if i == 0 else None) @ w[p + "o"].T
                h = rms(x, w[p + "n2"])
                choice = (h @ w[p + "router"].T).argmax(-1)
                f = torch.zeros_like(h)
                for t in range(T):
                    e = int(choice[t])
                    f[t] = w[f"{p}e{e}.w2"] @ torch.relu(w[f"{p}e{e}.w1"] @ h[t])
                x = x + f
            return rms(x, w["nf"]) @ w["emb"].T

        ref = [reference(r) for r in reqs]
        assert len({int(c) for c in (rms(w["emb"][reqs[0]], w["l0.n1"]) @ w["l0.router"].T).argmax(-1)}) > 1

        def whole(ids):
            s = eng.take_slot()
            try:
                return eng.step([StepEntry(s, ids, list(range(len(ids))))]).cpu()
            finally:
                eng.free_slot(s)

        alone = [whole(r) for r in reqs]
        for a, r in zip(alone, ref):
            assert rel_err(a, r) < FP32_VS_PLAIN
        # prompts of unequal lengths in one step, then one token each; twice, so that slots are used again
        for rnd in range(2):
            got, slots = replay.run_batches(eng_as_runtime(eng), reqs, 3, [5, 6, 12])
            for i in range(3):
                assert rel_err(got[i], ref[i]) < FP32_VS_PLAIN and rel_err(got[i], alone[i]) < SPLITS["float32"]
        assert eng.cache.slots.n_held == 0
    finally:
        unregister_part("feed_forward", "toy_top1_experts")
        unregister_part("position", "toy_learned_offset")
        unregister_part("position", "toy_distance_slopes")


@pytest.mark.parametrize("dtype,tol", [(torch.float32, FP32_VS_PLAIN), (torch.bfloat16, 3e-2)])
def test_a_position_encoding_that_biases_scores(dtype, tol):
    """A slope-times-distance bias on the scores (no rotation, nothing written into q or k), registered from
    outside: the mixer stores k and v itself, the attention kernels take the slopes, decode steps are
    captured (the part is graph-safe), and prompts cut in any way give the same logits."""
    from airframe_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from airframe_b200.engine import Engine, Model, StepEntry
    from airframe_b200.parts import known_parts, unregister_part
    from airframe_b200.weights import RandomSource, load_weights
    _register()
    try:
        assert "toy_distance_slopes" in known_parts("position")
        H, V, nq, nkv, hd, I, P = 64, 90, 4, 2, 16, 96, 200
        base = 2.0

        def norm(name):
            return PartSpec("rms_norm", {"weight": name, "size": H, "eps": 1e-6, "weight_offset": 1.0})

        layers = []
        for i in range(2):
            p = f"l{i}."
            mixer = PartSpec("attention", {"hidden_size": H, "num_heads": nq, "num_kv_heads": nkv, "head_dim": hd,
                                           "scale": 0.25, "softcap": 0.0, "window": 70 if i == 0 else None,
                                           "position": PartSpec("toy_distance_slopes", {"base": base, "heads": nq}),
                                           "q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "o_weight": p + "o"})
            ffn = PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "silu",
                                         "gate_weight": p + "g", "up_weight": p + "u", "down_weight": p + "d"})
            layers.append(LayerSpec(p, PartSpec("prenorm"), mixer, ffn,
                                    {"pre_mixer": norm(p + "n1"), "pre_feed_forward": norm(p + "n2")}))
        spec = ModelSpec("toy", H, V, P, PartSpec("token_embedding", {"weight": "emb", "vocab_size": V, "hidden_size": H,
                                                                      "scale": 1.0}),
                         layers, [ScheduleEntry(0), ScheduleEntry(1)], norm("nf"),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "softcap": 0.0, "tied_to": "emb"}))
        model = Model(spec, dtype, DEV)
        assert model.graph_safe
        decls = model.weight_decls()
        wts = load_weights(RandomSource(decls, 12, torch.bfloat16), decls, dtype, DEV)
        for i in range(2):                               # sharper scores, so that the bias decides something
            wts[f"l{i}.q"] = wts[f"l{i}.q"] * 20.0
        model.load(wts)
        eng = Engine(model, 64 * 12)
        w = {k: v.double().cpu() for k, v in wts.items()}

        def rms(x, wt):
            return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-6) * (1.0 + wt)

        def reference(ids):
            T = len(ids)
            x = w["emb"][ids]
            i_, j_ = torch.arange(T)[:, None], torch.arange(T)[None, :]
            for i in range(2):
                p = f"l{i}."
                h = rms(x, w[p + "n1"])
                q = (h @ w[p + "q"].T).reshape(T, nq, hd)
                k = (h @ w[p + "k"].T).reshape(T, nkv, hd)
                v = (h @ w[p + "v"].T).reshape(T, nkv, hd)
                mask = plain.visibility(T, 70 if i == 0 else None)
                ctx = torch.empty(T, nq, hd, dtype=torch.float64)
                for hh in range(nq):
                    sc = (q[:, hh] @ k[:, hh // (nq // nkv)].T) * 0.25 + base ** -(hh + 1) * (j_ - i_)
                    ctx[:, hh] = torch.softmax(sc.masked_fill(~mask, float("-inf")), -1) @ v[:, hh // (nq // nkv)]
                x = x + ctx.reshape(T, nq * hd) @ w[p + "o"].T
                h = rms(x, w[p + "n2"])
                g = h @ w[p + "g"].T
                x = x + ((g / (1 + torch.exp(-g))) * (h @ w[p + "u"].T)) @ w[p + "d"].T
            return rms(x, w["nf"]) @ w["emb"].T

        reqs = [replay.random_ids(V, n, 40 + n) for n in (150, 9, 75)]
        ref = [reference(r) for r in reqs]
        # the bias matters: without it the logits are others
        rt = eng_as_runtime(eng)
        alone = [replay.run_whole(rt, r) for r in reqs]
        for a, r in zip(alone, ref):
            assert rel_err(a, r) < tol
        tails = [replay.run_tail(rt, r, 8) for r in reqs]
        for t, a, r in zip(tails, alone, ref):
            assert rel_err(t, r) < tol
        assert eng.use_graphs and eng._graphs              # the decode steps ran as captured graphs
        got, _ = replay.run_batches(rt, reqs, 3, [100, 9, 20])
        for i in range(3):
            assert rel_err(got[i], ref[i]) < tol
        assert eng.cache.slots.n_held == 0
    finally:
        unregister_part("feed_forward", "toy_top1_experts")
        unregister_part("position", "toy_learned_offset")
        unregister_part("position", "toy_distance_slopes")


class eng_as_runtime:
    """What ``replay`` needs of a runtime, around a bare engine."""

    def __init__(self, engine):
        self.engine = engine

    def step(self, entries):
        return self.engine.step(entries)
