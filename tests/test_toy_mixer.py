"""A mixer with state of its own, defined here, is registered, built and
stepped without a change to the framework's files: a running average
h_t = d * h_{t-1} + (1 - d) * x_t W_in, y_t = h_t W_out, whose h lives in the
cache's per-sequence state.  The toy computes with torch (it is a test, not
the product); what is under test is the framework around it: registry,
weights, state storage and slots, schedule, step function."""
import pytest
import torch

import replay
from tolerances import rel_err

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def _register():
    from airframe_b200.parts import Mixer, StateNeed, register_part
    from airframe_b200.weights import WeightDecl

    @register_part("mixer", "toy_running_average")
    class RunningAverage(Mixer):
        def __init__(self, params, ctx):
            super().__init__(params, ctx)
            self.h, self.s, self.decay = params["hidden_size"], params["state_size"], params["decay"]
            self.p = params["prefix"]

        def state_need(self):
            return StateNeed((self.s,), "float32")

        def weight_decls(self):
            return [WeightDecl(self.p + "w_in", (self.s, self.h)), WeightDecl(self.p + "w_out", (self.h, self.s))]

        def load(self, weights):
            self.w_in = weights[self.p + "w_in"].float()
            self.w_out = weights[self.p + "w_out"].float()

        def forward(self, x, batch, view):
            u = x.float() @ self.w_in.T
            out = torch.empty_like(u)
            slots = batch.slots.tolist()
            starts = batch.seq_starts.tolist()
            for b, slot in enumerate(slots):
                h = view.state[slot]
                for t in range(starts[b], starts[b + 1]):
                    h = self.decay * h + (1 - self.decay) * u[t]
                    out[t] = h
                view.state[slot] = h
            return (out @ self.w_out.T).to(x.dtype)
    return RunningAverage


def test_toy_mixer_with_state_steps_through_the_engine():
    from airframe_b200.config import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
    from airframe_b200.engine import Engine, Model, StepEntry
    from airframe_b200.parts import known_parts, unregister_part
    from airframe_b200.weights import RandomSource, load_weights
    _register()
    try:
        assert "toy_running_average" in known_parts("mixer")
        H, V, S, I = 32, 50, 24, 64

        def norm(name):
            return PartSpec("rms_norm", {"weight": name, "size": H, "eps": 1e-6, "weight_offset": 1.0})

        def ffn(p):
            return PartSpec("gated_mlp", {"hidden_size": H, "intermediate_size": I, "activation": "gelu_tanh",
                                         "gate_weight": p + "g", "up_weight": p + "u", "down_weight": p + "d"})
        toy = PartSpec("toy_running_average", {"hidden_size": H, "state_size": S, "decay": 0.9, "prefix": "l0."})
        att = PartSpec("attention", {"hidden_size": H, "num_heads": 2, "num_kv_heads": 1, "head_dim": 16,
                                     "scale": 0.25, "softcap": 0.0, "window": 5,
                                     "position": PartSpec("rope", {"theta": 50.0, "rotary_dim": 16, "pairing": "half"}),
                                     "q_weight": "l1.q", "k_weight": "l1.k", "v_weight": "l1.v", "o_weight": "l1.o"})
        layers = [LayerSpec("l0.", PartSpec("prenorm"), toy, ffn("l0."),
                            {"pre_mixer": norm("l0.n1"), "pre_feed_forward": norm("l0.n2")}),
                  LayerSpec("l1.", PartSpec("prenorm"), att, ffn("l1."),
                            {"pre_mixer": norm("l1.n1"), "pre_feed_forward": norm("l1.n2")})]
        spec = ModelSpec("toy", H, V, 128, PartSpec("token_embedding", {"weight": "emb", "vocab_size": V,
                                                                        "hidden_size": H, "scale": 1.0}),
                         layers, [ScheduleEntry(0), ScheduleEntry(1)], norm("nf"),
                         PartSpec("lm_head", {"vocab_size": V, "hidden_size": H, "softcap": 0.0, "tied_to": "emb"}))
        model = Model(spec, torch.float32, DEV)
        decls = model.weight_decls()
        assert {"l0.w_in", "l0.w_out"} <= {d.name for d in decls}
        model.load(load_weights(RandomSource(decls, 1, torch.float32), decls, torch.float32, DEV))
        eng = Engine(model, 64 * 6)
        assert eng.cache.views[0].kv is None and tuple(eng.cache.views[0].state.shape[1:]) == (S,)
        assert eng.cache.views[1].state is None and eng.cache.views[1].kv is not None
        reqs = [replay.random_ids(V, n, 40 + n) for n in (30, 7, 19)]

        def whole(ids):
            s = eng.take_slot()
            try:
                return eng.step([StepEntry(s, ids, list(range(len(ids))))]).cpu()
            finally:
                eng.free_slot(s)

        ref = [whole(r) for r in reqs]
        assert not torch.allclose(ref[0][-1], whole(reqs[0][:-1] + [reqs[0][-1]])[0])   # positions differ
        # the state is carried: prompts of unequal lengths, then one token each, slots used again
        for rnd in range(2):
            slots = [eng.take_slot() for _ in reqs]
            fed = [5, 3, 10]
            out = eng.step([StepEntry(s, r[:f], list(range(f))) for s, r, f in zip(slots, reqs, fed)])
            pieces, o = [], 0
            for f in fed:
                pieces.append([out[o:o + f].cpu()])
                o += f
            live = [0, 1, 2]
            while live:
                out = eng.step([StepEntry(slots[i], [reqs[i][fed[i]]], [0]) for i in live])
                for r, i in enumerate(live):
                    pieces[i].append(out[r:r + 1].cpu())
                    fed[i] += 1
                for i in [i for i in live if fed[i] >= len(reqs[i])]:
                    eng.free_slot(slots[i])
                    live.remove(i)
            for i in range(3):
                assert rel_err(torch.cat(pieces[i]), ref[i]) < 2e-5, (rnd, i)
        # a slot that is taken again starts from zero state
        s = eng.take_slot()
        assert float(eng.cache.views[0].state[s].abs().sum()) == 0
        eng.free_slot(s)
    finally:
        unregister_part("mixer", "toy_running_average")
