"""Schedules of the Gemma-2 2B sizes that the small engine tests do not reach, against the plain
implementation in 32-bit and bfloat16: the real window (a ring of 64 pages) lapped by one prompt and
crossed while decoding; decode batches of forty unequal sequences (the captured step of 48 rows, the
64-token product tile, one split a sequence); positions up to the 8,192nd; the real vocabulary."""
import pytest
import torch

import plain_gemma2 as plain
import replay
from tiny import WIDE_D, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["float32", "bfloat16"])
def dtype(request):
    return request.param


def load(folder, dtype, max_tokens, **kw):
    from airframe_b200.engine import GpuRuntime
    return GpuRuntime.load(folder, dtype=dtype, max_tokens=max_tokens, **kw)


# ---------------------------------------------------------------- the real window

REAL_WINDOW = dict(WIDE_D, sliding_window=4096, max_position_embeddings=8192)


@pytest.fixture(scope="module")
def window_case(tmp_path_factory):
    folder = make_folder(REAL_WINDOW, seed=21, store_dtype="bfloat16", root=tmp_path_factory.mktemp("w4096"))
    cfg, w = plain.read_model_folder(folder)
    ids = replay.random_ids(cfg["vocab_size"], 4308, 77)
    x = plain.hidden_states(cfg, w, ids)
    tail = list(range(4080, 4308))
    ref = plain.lm_head(x[tail], cfg, w)            # logits at positions 4080..4307
    return {"folder": folder, "ids": ids, "ref": ref, "first": tail[0]}


def test_a_prompt_that_laps_the_ring_in_one_step(window_case, dtype):
    """4,300 tokens in one step: the local layer's ring of 4,096 rows keeps the last of the rows that
    share a place; then 8 single tokens read it."""
    from airframe_b200.engine import StepEntry
    rt = load(window_case["folder"], dtype, 64 * 70, max_context=8192)
    ids, ref, first = window_case["ids"], window_case["ref"], window_case["first"]
    s = rt.engine.take_slot()
    try:
        want = [4090, 4095, 4096, 4097, 4299]
        got = [rt.step([StepEntry(s, ids[:4300], want)]).cpu()]
        for t in ids[4300:4308]:
            got.append(rt.step([StepEntry(s, [t], [0])]).cpu())
        got = torch.cat(got)
        rows = [p - first for p in want] + [p - first for p in range(4300, 4308)]
        assert rel_err(got, ref[rows]) < VS_PLAIN[dtype]
    finally:
        rt.engine.free_slot(s)


def test_decoding_across_the_window(window_case, dtype):
    """4,090 tokens of prompt, then one token a step across position 4,096, where the ring wraps and
    the window starts to cut the first keys off."""
    from airframe_b200.engine import StepEntry
    rt = load(window_case["folder"], dtype, 64 * 70, max_context=8192)
    ids, ref, first = window_case["ids"], window_case["ref"], window_case["first"]
    s = rt.engine.take_slot()
    try:
        got = [rt.step([StepEntry(s, ids[:4090], [4089])]).cpu()]
        for t in ids[4090:4110]:
            got.append(rt.step([StepEntry(s, [t], [0])]).cpu())
        got = torch.cat(got)
        rows = [p - first for p in range(4089, 4110)]
        assert rel_err(got, ref[rows]) < VS_PLAIN[dtype]
        # every single position, not only the worst: the wrap is at one of them
        for g, r in zip(got, ref[rows]):
            assert rel_err(g, r) < VS_PLAIN[dtype]
    finally:
        rt.engine.free_slot(s)


# ---------------------------------------------------------------- forty sequences in a decode step

@pytest.fixture(scope="module")
def many_case(tmp_path_factory):
    folder = make_folder(WIDE_D, seed=22, store_dtype="bfloat16", root=tmp_path_factory.mktemp("many"))
    cfg, w = plain.read_model_folder(folder)
    lens = [3 + (37 * i) % 180 for i in range(40)]          # 3 .. 182 tokens, all different enough
    reqs = [replay.random_ids(cfg["vocab_size"], n + 6, 900 + i) for i, n in enumerate(lens)]
    ref = [plain.logits(cfg, w, r)[n - 1:] for r, n in zip(reqs, lens)]     # the last prompt row and 6 decoded
    return {"folder": folder, "lens": lens, "reqs": reqs, "ref": ref}


def test_decode_batch_of_forty_unequal_sequences(many_case, dtype):
    from airframe_b200.engine import Engine, StepEntry
    rt = load(many_case["folder"], dtype, 64 * 40 * 4, max_sequences=64)
    eng = rt.engine
    lens, reqs, ref = many_case["lens"], many_case["reqs"], many_case["ref"]
    slots = [eng.take_slot() for _ in reqs]
    try:
        got = [[] for _ in reqs]
        lg = rt.step([StepEntry(s, r[:n], [n - 1]) for s, r, n in zip(slots, reqs, lens)]).cpu()
        for i in range(40):
            got[i].append(lg[i])
        for k in range(6):
            lg = rt.step([StepEntry(s, [r[n + k]], [0]) for s, r, n in zip(slots, reqs, lens)]).cpu()
            for i in range(40):
                got[i].append(lg[i])
        if eng.use_graphs:
            assert Engine.padded_batch(40) == 48 and 48 in eng._graphs      # the captured step of 48 rows ran
        worst = max(rel_err(torch.stack(g), r) for g, r in zip(got, ref))
        assert worst < VS_PLAIN[dtype], worst
    finally:
        for s in slots:
            eng.free_slot(s)


# ---------------------------------------------------------------- the last positions of the context

# head size 256 as at 2B sizes, narrow otherwise: what is tried here is positions, pages and splits
LONG = dict(WIDE_D, hidden_size=256, num_attention_heads=2, num_key_value_heads=1, intermediate_size=512,
            vocab_size=512, sliding_window=4096, max_position_embeddings=8192)


@pytest.fixture(scope="module")
def long_case(tmp_path_factory):
    folder = make_folder(LONG, seed=23, store_dtype="bfloat16", root=tmp_path_factory.mktemp("long"))
    cfg, w = plain.read_model_folder(folder)
    ids = replay.random_ids(cfg["vocab_size"], 8192, 78)
    x = plain.hidden_states(cfg, w, ids)
    ref = plain.lm_head(x[7990:], cfg, w)
    return {"folder": folder, "ids": ids, "ref": ref}


def test_positions_up_to_the_end_of_the_context(long_case, dtype):
    """A prompt of 8,000 tokens, then single tokens up to the 8,192nd: rotary angles of large positions
    in 32 bits, page tables of 128 pages, a sequence cut into many splits."""
    from airframe_b200.cache import ContextOverflow
    from airframe_b200.engine import StepEntry
    rt = load(long_case["folder"], dtype, 8192 + 64, max_context=8192, max_sequences=2)
    ids, ref = long_case["ids"], long_case["ref"]
    s = rt.engine.take_slot()
    try:
        got = [rt.step([StepEntry(s, ids[:8000], list(range(7990, 8000)))]).cpu()]
        for t in ids[8000:8192]:
            got.append(rt.step([StepEntry(s, [t], [0])]).cpu())
        got = torch.cat(got)
        assert got.shape == ref.shape
        assert rel_err(got, ref) < VS_PLAIN[dtype]
        assert rel_err(got[-8:], ref[-8:]) < VS_PLAIN[dtype]
        assert rt.engine.length(s) == 8192
        with pytest.raises(ContextOverflow):
            rt.step([StepEntry(s, [1], [0])])
    finally:
        rt.engine.free_slot(s)


# ---------------------------------------------------------------- the real vocabulary

def test_head_at_the_real_vocabulary(dtype, tmp_path):
    """256,000 rows in the head (2,000 weight tiles: the product's many-wave variant in bfloat16, the
    plain product in 32-bit), two layers, a 24-token prompt and two decoded tokens."""
    from airframe_b200.engine import StepEntry
    cfg_dict = dict(WIDE_D, vocab_size=256000)
    folder = make_folder(cfg_dict, seed=24, store_dtype="bfloat16", root=tmp_path / "v256k")
    cfg, w = plain.read_model_folder(folder)
    ids = replay.random_ids(cfg["vocab_size"], 26, 79)
    ref = plain.logits(cfg, w, ids)
    rt = load(folder, dtype, 128)
    s = rt.engine.take_slot()
    try:
        got = [rt.step([StepEntry(s, ids[:24], list(range(24)))]).cpu()]
        for t in ids[24:]:
            got.append(rt.step([StepEntry(s, [t], [0])]).cpu())
        got = torch.cat(got)
        assert got.shape == (26, 256000)
        assert rel_err(got, ref) < VS_PLAIN[dtype]
        # the arg-max is the same token wherever the reference's own margin allows it
        top2 = ref.topk(2, dim=-1).values
        clear = (top2[:, 0] - top2[:, 1]) > 4 * VS_PLAIN[dtype] * ref.abs().max()
        assert bool((got.argmax(-1)[clear] == ref.argmax(-1)[clear]).all())
    finally:
        rt.engine.free_slot(s)
