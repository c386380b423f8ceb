"""Generation through the programming entry point and the command line."""
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_gemma2 as plain
import replay
from tiny import CONFIGS, make_folder

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module", params=["A", "B"])
def case(request, tmp_path_factory):
    name = request.param
    store = "float32"
    folder = make_folder(CONFIGS[name], seed=21, store_dtype=store, root=tmp_path_factory.mktemp(name))
    cfg, w = plain.read_model_folder(folder)
    return name, folder, cfg, w


def test_greedy_generation_equals_the_plain_chain(case):
    """The tiny configurations' own workloads: A prompts 5/11/17 then 8 tokens, B prompts 1/9/20/33 then 12."""
    from airframe_b200.engine import GpuRuntime
    from airframe_b200.sampling import SamplingParams
    name, folder, cfg, w = case
    lens, n_new = ([5, 11, 17], 8) if name == "A" else ([1, 9, 20, 33], 12)
    prompts = [replay.random_ids(cfg["vocab_size"], n, 7 + n) for n in lens]
    rt = GpuRuntime.load(folder, dtype="float32", max_tokens=64 * 8)
    params = SamplingParams(max_tokens=n_new, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    got = rt.generate(prompts, params)
    want = [plain.generate_greedy(cfg, w, p, n_new) for p in prompts]
    assert got == want
    assert rt.generate(prompts[1], params) == want[1]                   # one request alone, flat ids
    # stop tokens: the model's own end token stops a sequence, the token is not emitted
    stop = want[0][3]
    cut = want[0][: want[0].index(stop)]
    got = rt.generate(prompts, SamplingParams(max_tokens=n_new, temperature=0.0, repetition_penalty=1.0,
                                              ignore_eos=True, stop_token_ids=[stop]))
    assert got[0] == cut
    for g, wnt in zip(got[1:], want[1:]):
        assert g == (wnt[: wnt.index(stop)] if stop in wnt else wnt)
    assert rt.engine.cache.slots.n_held == 0
    assert rt.eos_token() == (1 if name == "A" else 3)


def test_temperature_sampling_is_seeded_and_batch_independent(case):
    from airframe_b200.engine import GpuRuntime
    from airframe_b200.sampling import SamplingParams
    name, folder, cfg, w = case
    prompts = [replay.random_ids(cfg["vocab_size"], n, 70 + n) for n in (5, 11, 17)]
    rt = GpuRuntime.load(folder, dtype="bfloat16", max_tokens=64 * 8)
    p = SamplingParams(max_tokens=8, temperature=0.8, ignore_eos=True)    # reference defaults otherwise
    a = rt.generate(prompts, p)
    assert a == rt.generate(prompts, p)                                   # same seed, same tokens
    assert a != rt.generate(prompts, SamplingParams(max_tokens=8, temperature=0.8, ignore_eos=True, seed=43))
    assert rt.generate(prompts[0], p) == a[0]                             # the first request alone
    assert all(len(x) == 8 and all(0 <= t < cfg["vocab_size"] for t in x) for x in a)


def test_the_device_a_step_ahead_of_the_host_gives_the_same_tokens(case):
    from airframe_b200.engine import GpuRuntime
    from airframe_b200.sampling import SamplingParams
    name, folder, cfg, w = case
    prompts = [replay.random_ids(cfg["vocab_size"], n, 90 + n) for n in (4, 13, 2, 9, 6)]
    rt = GpuRuntime.load(folder, dtype="bfloat16", max_tokens=64 * 8)
    free = SamplingParams(max_tokens=10, temperature=0.9, top_p=0.95, repetition_penalty=1.0, ignore_eos=True, seed=5)
    rt.generate(prompts[0], free)                                         # (makes the loop)
    runs = {}
    for ahead in (False, True):
        rt._loop.pipelined = ahead
        a = rt.generate(prompts, free)
        # tokens that some sequences emit midway become stop tokens: those sequences end early, one step late for the host
        stops = [a[0][4], a[2][7], a[3][0]]
        b = rt.generate(prompts, SamplingParams(max_tokens=10, temperature=0.9, top_p=0.95, repetition_penalty=1.0,
                                                ignore_eos=True, seed=5, stop_token_ids=stops))
        runs[ahead] = (a, b, list(rt._loop.finish_reasons))
        assert rt.engine.cache.slots.n_held == 0
    assert runs[False] == runs[True]
    assert "stop" in runs[True][2] and len(runs[True][1][3]) == 0


def test_more_requests_than_fit_one_batch(case):
    from airframe_b200.engine import GpuRuntime
    from airframe_b200.sampling import SamplingParams
    name, folder, cfg, w = case
    prompts = [replay.random_ids(cfg["vocab_size"], 3 + i, 200 + i) for i in range(7)]
    rt = GpuRuntime.load(folder, dtype="float32", max_tokens=64 * 3)      # three pages: three requests at a time
    params = SamplingParams(max_tokens=4, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    got = rt.generate(prompts, params)
    assert rt._loop.batches_run == [[0, 1, 2], [3, 4, 5], [6]]
    assert got == [plain.generate_greedy(cfg, w, p, 4) for p in prompts]


def test_command_line(case):
    name, folder, cfg, w = case
    prompt = replay.random_ids(cfg["vocab_size"], 6, 5)
    want = plain.generate_greedy(cfg, w, prompt, 5)
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "simple_flight"), "--model", str(folder),
                          "--dtype", "float32", "--max-tokens", "5", "--ignore-eos",
                          ",".join(map(str, prompt))], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr
    assert "Output: " + " ".join(map(str, want)) in out.stdout and "Flight Complete." in out.stdout
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "simple_flight"), "1,2"], capture_output=True,
                         text=True, env={"PATH": "/usr/bin:/bin"}, timeout=600)
    assert out.returncode != 0 and "LIBSHIMMY_MODEL_PATH" in out.stderr


def test_command_line_with_a_named_random_model():
    """--random NAME runs a preset with seeded weights; two --prompt-ids make a batch; the same seed gives
    the same tokens."""
    runs = []
    for _ in range(2):
        out = subprocess.run([sys.executable, str(ROOT / "bin" / "simple_flight"), "--random", "tinyB", "--seed", "5",
                              "--dtype", "fp32", "--max-tokens", "6", "--ignore-eos", "--prompt-ids", "3,4,5",
                              "--prompt-ids", "9"], capture_output=True, text=True, timeout=600)
        assert out.returncode == 0, out.stderr
        lines = [ln for ln in out.stdout.splitlines() if ln.startswith("Output ")]
        assert len(lines) == 2 and all(len(ln.split(":")[1].split()) == 6 for ln in lines)
        runs.append(lines)
    assert runs[0] == runs[1]
    out = subprocess.run([sys.executable, str(ROOT / "bin" / "simple_flight"), "--random", "nope"], capture_output=True,
                         text=True, timeout=600)
    assert out.returncode != 0 and "unknown preset" in out.stderr


def test_runtime_refuses_the_cpu(case):
    from airframe_b200.engine import GpuRuntime
    with pytest.raises(RuntimeError, match="CUDA device only"):
        GpuRuntime.load(case[1], device="cpu")


@pytest.mark.parametrize("name", ["D", "C"])
def test_greedy_tokens_from_the_head_equal_those_from_the_logits(name, tmp_path):
    """bfloat16, sizes whose head runs on the tensor cores (D) and sizes whose head does not (C): generation with
    the arg-max found in the head's epilogue gives the tokens that sampling the written logits gives, and the
    step function's own greedy answer equals the arg-max of its logits."""
    from airframe_b200.engine import GpuRuntime, StepEntry
    from airframe_b200.sampling import SamplingParams
    folder = make_folder(CONFIGS[name], seed=33, store_dtype="bfloat16", root=tmp_path / "m")
    cfg, _ = plain.read_model_folder(folder)
    prompts = [replay.random_ids(cfg["vocab_size"], n, 50 + n) for n in (7, 70, 33)]
    rt = GpuRuntime.load(folder, dtype="bfloat16", max_tokens=64 * 8)
    params = SamplingParams(max_tokens=10, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    fused = rt.generate(prompts, params)
    rt.engine.fused_greedy = False                      # the loop then samples the logits it is given
    try:
        assert rt.generate(prompts, params) == fused
    finally:
        rt.engine.fused_greedy = True
    slots = [rt.engine.take_slot() for _ in prompts]
    try:
        toks = rt.engine.step([StepEntry(s, p, [0, len(p) - 1]) for s, p in zip(slots, prompts)], greedy=True)
        for s in slots:
            rt.engine.free_slot(s)
        slots = [rt.engine.take_slot() for _ in prompts]
        logits = rt.engine.step([StepEntry(s, p, [0, len(p) - 1]) for s, p in zip(slots, prompts)])
        assert toks.dtype == torch.int32 and toks.tolist() == logits.argmax(-1).tolist()
    finally:
        for s in slots:
            rt.engine.free_slot(s)
