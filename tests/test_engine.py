"""The engine against the plain implementation, in 32-bit and bfloat16, under
every way of cutting the work: whole requests, the last 32 tokens one by one,
batches of unequal lengths one after another (slots used again), long
decoding, and the first tokens of a sequence."""
import pytest
import torch

import plain_gemma2 as plain
import replay
from tiny import CONFIGS, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err

pytestmark = pytest.mark.gpu

# request lengths: some cross the window in the prompt, some while decoding,
# some wrap the ring of the local layers (64 rows for all three windows)
LENGTHS = {"A": [5, 11, 17, 40, 64, 1, 33], "B": [1, 9, 20, 33, 100, 128, 70], "C": [3, 45, 130, 300, 65, 64, 200],
           "D": [70, 5, 210, 129, 64, 101, 33], "E": [70, 5, 150, 129, 64, 101, 33], "F": [66, 5, 140, 129, 64, 101, 33], "G": [3, 45, 130, 200, 65, 64, 100]}
PROMPTS = {"A": [5, 3, 17, 10, 20, 1, 9], "B": [1, 9, 5, 33, 40, 60, 17], "C": [3, 39, 41, 150, 2, 64, 63],
           "D": [40, 5, 99, 128, 1, 100, 20], "E": [40, 5, 99, 128, 1, 100, 20], "F": [40, 5, 99, 128, 1, 100, 20], "G": [3, 39, 41, 150, 2, 64, 63]}


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E", "F", "G"])
def case(request, tmp_path_factory):
    name = request.param
    folder = make_folder(CONFIGS[name], seed=11, store_dtype="bfloat16", root=tmp_path_factory.mktemp(name))
    cfg, w = plain.read_model_folder(folder)
    reqs = [replay.random_ids(cfg["vocab_size"], n, 100 + i) for i, n in enumerate(LENGTHS[name])]
    ref = [plain.logits(cfg, w, r) for r in reqs]
    return {"name": name, "folder": folder, "cfg": cfg, "requests": reqs, "plain": ref, "rt": {}, "whole": {}}


@pytest.fixture(params=["float32", "bfloat16"])
def dtype(request):
    return request.param


def runtime(case, dtype):
    from airframe_b200.engine import GpuRuntime
    if dtype not in case["rt"]:
        case["rt"][dtype] = GpuRuntime.load(case["folder"], dtype=dtype, max_tokens=64 * 24)
    return case["rt"][dtype]


def whole(case, dtype):
    if dtype not in case["whole"]:
        rt = runtime(case, dtype)
        case["whole"][dtype] = [replay.run_whole(rt, r) for r in case["requests"]]
    return case["whole"][dtype]


def test_each_request_alone_and_whole(case, dtype):
    for got, ref in zip(whole(case, dtype), case["plain"]):
        assert got.shape == ref.shape and got.dtype == torch.float32
        assert rel_err(got, ref) < VS_PLAIN[dtype]


def test_last_32_tokens_one_by_one(case, dtype):
    rt = runtime(case, dtype)
    for ids, w, ref in zip(case["requests"], whole(case, dtype), case["plain"]):
        if len(ids) < 2:
            continue
        got = replay.run_tail(rt, ids, 32)
        assert rel_err(got, ref) < VS_PLAIN[dtype]
        assert rel_err(got, w) < SPLITS[dtype]


def test_batches_of_unequal_lengths_with_slots_used_again(case, dtype):
    rt = runtime(case, dtype)
    got, slots = replay.run_batches(rt, case["requests"], 3, PROMPTS[case["name"]])
    assert slots[0] == slots[1] == [0, 1, 2] and slots[2] == [0]          # the same slots serve every batch
    for i, (w, ref) in enumerate(zip(whole(case, dtype), case["plain"])):
        assert got[i].shape == ref.shape
        assert rel_err(got[i], ref) < VS_PLAIN[dtype], f"request {i}"
        assert rel_err(got[i], w) < SPLITS[dtype], f"request {i}"
    held = rt.engine.cache.pages_held()
    assert all(n == 0 for n in held.values()) and rt.engine.cache.slots.n_held == 0


def test_long_decoding_from_the_first_token(case, dtype):
    """One token of prompt, everything else decoded: the first tokens of a
    sequence and a long run of single-token steps."""
    rt = runtime(case, dtype)
    i = max(range(len(case["requests"])), key=lambda j: len(case["requests"][j]))
    ids, ref = case["requests"][i], case["plain"][i]
    got = replay.run_tail(rt, ids, len(ids) - 1)
    assert rel_err(got[:4], ref[:4]) < VS_PLAIN[dtype]
    assert rel_err(got, ref) < VS_PLAIN[dtype]
    assert rel_err(got, whole(case, dtype)[i]) < SPLITS[dtype]


def test_results_do_not_depend_on_batch_mates_or_slots(case, dtype):
    rt = runtime(case, dtype)
    reqs = case["requests"]
    a, _ = replay.run_batches(rt, reqs[:4], 4, [len(r) for r in reqs[:4]])
    # other mates, other slots: hold two slots so the requests land elsewhere
    hold = [rt.engine.take_slot(), rt.engine.take_slot()]
    try:
        b, slots = replay.run_batches(rt, [reqs[3], reqs[1], reqs[6]], 3, [len(reqs[3]), len(reqs[1]), len(reqs[6])])
    finally:
        for s in hold:
            rt.engine.free_slot(s)
    assert slots[0] == [2, 3, 4]
    assert rel_err(b[0], a[3]) < SPLITS[dtype] and rel_err(b[1], a[1]) < SPLITS[dtype]


def test_the_same_work_gives_the_same_bits(case, dtype):
    """No kernel adds in an order that depends on timing: a request run twice, and the same batch run
    twice through the captured decode step, give bitwise equal logits."""
    rt = runtime(case, dtype)
    ids = case["requests"][2]
    a, b = replay.run_whole(rt, ids), replay.run_whole(rt, ids)
    assert torch.equal(a, b)
    a, b = replay.run_tail(rt, ids, 16), replay.run_tail(rt, ids, 16)
    assert torch.equal(a, b)


def test_decode_steps_fed_from_the_device(case, dtype):
    """``decode_rows``: the step's tokens lie on the device, rows keep their places and a row may be
    unused; the logits are those of the same step fed from the host."""
    from airframe_b200.engine import StepEntry, StepError
    rt = runtime(case, dtype)
    eng = rt.engine
    reqs = [r for r in case["requests"] if len(r) >= 5][:3]
    outs = {}
    for way in ("host", "device"):
        slots = [eng.take_slot() for _ in reqs]
        try:
            eng.step([StepEntry(s, r[:-3], []) for s, r in zip(slots, reqs)])
            got = []
            for k in (3, 2, 1):                                  # the last three tokens, one step each
                toks = [r[len(r) - k] for r in reqs]
                live = [0, 2] if k == 1 else [0, 1, 2]           # the middle row is unused in the last step
                if way == "host":
                    lg = eng.step([StepEntry(slots[i], [toks[i]], [0]) for i in live])
                    got.append(lg.clone())
                else:
                    dev = torch.tensor(toks, dtype=torch.int32, device=eng.device)
                    lg = eng.decode_rows([slots[i] if i in live else None for i in range(3)], dev)
                    got.append(lg[live].clone())
                    # the same step again on its own inputs changes nothing: not these logits, not the steps after
                    eng.repeat_last_decode(2)
                    assert torch.equal(lg[live], got[-1])
            outs[way] = got
        finally:
            for s in slots:
                eng.free_slot(s)
    for a, b in zip(outs["host"], outs["device"]):
        assert a.shape == b.shape and rel_err(b, a) < SPLITS[dtype]
    s = eng.take_slot()
    try:
        dev = torch.zeros(2, dtype=torch.int32, device=eng.device)
        with pytest.raises(StepError, match="tokens in the cache"):
            eng.decode_rows([s, None], dev)
        with pytest.raises(StepError, match="at least one sequence"):
            eng.decode_rows([None, None], dev)
        eng.step([StepEntry(s, [1, 2], [])])
        with pytest.raises(StepError, match="int32"):
            eng.decode_rows([s], dev.float())
        with pytest.raises(StepError, match="each slot once"):
            eng.decode_rows([s, s], dev)
    finally:
        eng.free_slot(s)


def test_step_errors(case):
    from airframe_b200.cache import CacheFull, ContextOverflow
    from airframe_b200.engine import StepEntry, StepError
    rt = runtime(case, "float32")
    V = case["cfg"]["vocab_size"]
    s, t = rt.engine.take_slot(), rt.engine.take_slot()
    try:
        with pytest.raises(StepError, match="not held"):
            rt.step([StepEntry(17, [1], [0])])
        with pytest.raises(StepError, match="outside the vocabulary"):
            rt.step([StepEntry(s, [V], [0])])
        with pytest.raises(StepError, match="wanted place"):
            rt.step([StepEntry(s, [1, 2], [2])])
        with pytest.raises(StepError, match="twice"):
            rt.step([StepEntry(s, [1], []), StepEntry(s, [1], [])])
        with pytest.raises(StepError, match="at least one token"):
            rt.step([StepEntry(s, [], [])])
        assert rt.step([StepEntry(s, [1, 2, 3], [])]) is None            # nothing wanted
        with pytest.raises(StepError, match="either all start or all go on"):
            rt.step([StepEntry(s, [1], [0]), StepEntry(t, [1], [0])])
        with pytest.raises(StepError, match="one token each"):
            rt.step([StepEntry(s, [1, 2], [0])])
        with pytest.raises(ContextOverflow):
            rt.step([StepEntry(t, [1] * (case["cfg"]["max_position_embeddings"] + 1), [])])
        assert rt.engine.length(s) == 3 and rt.engine.length(t) == 0     # failed steps change nothing
    finally:
        rt.engine.free_slot(s)
        rt.engine.free_slot(t)


@pytest.mark.parametrize("name", ["D", "F", "H"])
def test_projection_with_the_rotary_epilogue_switched_on(name, tmp_path):
    """The attention part's option ``rope_epilogue`` (rotation and cache write in the projection's epilogue):
    whole prompts, decoding (split-K: the last block adds the parts) and batches give the plain logits."""
    from airframe_b200.engine import GpuRuntime

    def on(spec):
        for layer in spec.layers:
            layer.mixer.params["rope_epilogue"] = True

    folder = make_folder(CONFIGS[name], seed=13, store_dtype="bfloat16", root=tmp_path / "m")
    cfg, w = plain.read_model_folder(folder)
    rt = GpuRuntime.load(folder, dtype="bfloat16", max_tokens=64 * 24, spec_edit=on)
    assert all(b.mixer.rope_epilogue for b in rt.model.blocks)
    reqs = [replay.random_ids(cfg["vocab_size"], n, 400 + n) for n in (150, 9, 70)]
    ref = [plain.logits(cfg, w, r) for r in reqs]
    for r, want in zip(reqs, ref):
        assert rel_err(replay.run_whole(rt, r), want) < VS_PLAIN["bfloat16"]
        assert rel_err(replay.run_tail(rt, r, 8), want) < VS_PLAIN["bfloat16"]
    got, _ = replay.run_batches(rt, reqs, 3, [100, 9, 20])
    for i, want in enumerate(ref):
        assert rel_err(got[i], want) < VS_PLAIN["bfloat16"]
