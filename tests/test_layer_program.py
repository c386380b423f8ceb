"""The layers of a decode step as one kernel (``csrc/decode_layers.cu``, opt-in)
against the plain implementation and against the chain of kernels: the last
tokens one by one, batches of unequal lengths whose padding rows and freed
slots it must ignore, and a model whose sizes it refuses (the chain serves)."""
import pytest
import torch

import plain_gemma2 as plain
import replay
from tiny import CONFIGS, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err

LENGTHS = [70, 5, 210, 129, 64, 101, 33]
PROMPTS = [40, 5, 99, 128, 1, 100, 20]


def test_k_parts_keep_the_blocks_busy():
    from airframe_b200.engine.layer_program import plan_k_parts
    from airframe_b200.parts import NotFusable
    # 72 row tiles of K = 9216 on 148 blocks: parts of at most 3584 columns, two rounds of 2304
    assert plan_k_parts(72, 9216, 148, 3584) == 4
    assert plan_k_parts(72, 2048, 148, 3584) == 2
    assert plan_k_parts(6, 384, 148, 3584) == 3
    # an epilogue that needs whole rows takes one part or nothing
    assert plan_k_parts(128, 2304, 148, 3584, fixed_one=True) == 1
    with pytest.raises(NotFusable):
        plan_k_parts(128, 4608, 148, 3584, fixed_one=True)
    with pytest.raises(NotFusable):
        plan_k_parts(10, 100, 148, 3584)          # no multiple of 64


@pytest.fixture(scope="module", params=["H", "D"])
def case(request, tmp_path_factory):
    from airframe_b200.engine import GpuRuntime
    name = request.param
    folder = make_folder(CONFIGS[name], seed=13, store_dtype="bfloat16", root=tmp_path_factory.mktemp(name))
    cfg, w = plain.read_model_folder(folder)
    reqs = [replay.random_ids(cfg["vocab_size"], n, 300 + i) for i, n in enumerate(LENGTHS)]
    rt = GpuRuntime.load(folder, dtype="bfloat16", max_tokens=64 * 24)
    whole = [replay.run_whole(rt, r) for r in reqs]                  # prompts never use the one-kernel path
    rt.engine.model.fuse_decode = True
    return {"rt": rt, "requests": reqs, "plain": [plain.logits(cfg, w, r) for r in reqs], "whole": whole}


def fused_programs(rt):
    return [p for p in rt.engine.model._programs.values() if p is not None]


@pytest.mark.gpu
def test_last_32_tokens_one_by_one_in_one_kernel(case):
    from airframe_b200 import kernels
    rt = case["rt"]
    for ids, w, ref in zip(case["requests"], case["whole"], case["plain"]):
        got = replay.run_tail(rt, ids, 32)
        assert rel_err(got, ref) < VS_PLAIN["bfloat16"]
        assert rel_err(got, w) < SPLITS["bfloat16"]
    assert fused_programs(rt), rt.engine.model.not_fused_because
    kernels.check_device_errors(rt.engine.device)


@pytest.mark.gpu
def test_batches_of_unequal_lengths_in_one_kernel(case):
    from airframe_b200 import kernels
    rt = case["rt"]
    for _ in range(2):                                               # slots and pages are used again
        got, slots = replay.run_batches(rt, case["requests"], 3, PROMPTS)
        for i, (w, ref) in enumerate(zip(case["whole"], case["plain"])):
            assert rel_err(got[i], ref) < VS_PLAIN["bfloat16"], f"request {i}"
            assert rel_err(got[i], w) < SPLITS["bfloat16"], f"request {i}"
    assert {p.n_tok for p in fused_programs(rt)} >= {1, 4}            # batches of 3 are padded to 4 rows
    assert rt.engine.cache.slots.n_held == 0
    kernels.check_device_errors(rt.engine.device)


@pytest.mark.gpu
def test_the_same_step_twice_gives_the_same_bits(case):
    from airframe_b200.engine import StepEntry
    rt = case["rt"]
    eng = rt.engine
    outs = []
    for _ in range(2):
        slots = [eng.take_slot() for _ in range(3)]
        eng.step([StepEntry(s, r[:n], []) for s, r, n in zip(slots, case["requests"][2:5], (150, 90, 40))])
        outs.append(eng.step([StepEntry(s, [r[n]], [0]) for s, r, n in zip(slots, case["requests"][2:5], (150, 90, 40))]).clone())
        for s in slots:
            eng.free_slot(s)
    assert torch.equal(outs[0], outs[1])


@pytest.mark.gpu
def test_sizes_the_one_kernel_step_refuses_run_as_a_chain(tmp_path):
    from airframe_b200.engine import GpuRuntime
    folder = make_folder(CONFIGS["C"], seed=3, store_dtype="bfloat16", root=tmp_path)
    cfg, w = plain.read_model_folder(folder)
    rt = GpuRuntime.load(folder, dtype="bfloat16", max_tokens=64 * 8)
    rt.engine.model.fuse_decode = True
    ids = replay.random_ids(cfg["vocab_size"], 50, 1)
    got = replay.run_tail(rt, ids, 8)
    assert rel_err(got, plain.logits(cfg, w, ids)) < VS_PLAIN["bfloat16"]
    assert not fused_programs(rt) and "head_dim" in rt.engine.model.not_fused_because


def test_decode_attention_split_counts():
    """The grid's third extent: the count that equal lengths use, with room above it for a long
    sequence among short ones, never more than the pages there are."""
    from airframe_b200 import kernels as K
    for batch, nkv in ((1, 4), (8, 4), (16, 4), (16, 8), (64, 4), (128, 16)):
        for ctx, window in ((8192, 0), (2048, 4096), (100, 0), (8192, 512)):
            equal = K.attn_decode_splits(batch, nkv, ctx, window)
            most = K.attn_decode_max_splits(batch, nkv, ctx, window)
            rows = min(ctx, window) if window else ctx
            pages = (rows + 63) // 64 + (1 if window else 0)
            assert 1 <= equal <= most <= max(1, min(pages, 64))
            assert batch * nkv * most <= max(3 * 148, batch * nkv * equal, batch * nkv)
    assert K.attn_decode_max_splits(8, 4, 8192, 0) == 13 and K.attn_decode_splits(8, 4, 8192, 0) == 4
    assert K.attn_decode_max_splits(64, 4, 8192, 0) == 1
