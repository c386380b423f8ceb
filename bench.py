#!/usr/bin/env python3
"""Decode and prefill throughput of Gemma-2 2B sizes (random weights, bf16) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences that hold 2,048-token
prompts (context limit 8192): the model's step function with the greedy choice in
its head's epilogue, stepped as the generation loop steps it (a step takes its
tokens from the device and is queued before the host has read them).  ``value`` is decoded
tokens a second, timed with CUDA events around exactly K steps after W warm-up
steps (default 32; whatever W is, the first decode step is run 64 more times on its own
inputs before the warm-up goes on: the first 30 or so steps after a burst of prompts run at
lowered clocks, about 2.1 ms instead of 1.8).  ``e2e`` is the same through
``GpuRuntime.generate`` with host token lists in and out: max(W, 32) + K + 1 tokens a sequence, the
clock on the last K steps.  The line also carries
the prefill rate of 2,048 tokens with its fraction of the bf16 peak (and, under ``profiled``,
the same for its products and its attention kernels apart, from a run under a profiler), the decode
step's fraction of the HBM roofline, decode at batch 1 and 64, the clocks seen
during the timed region and the number of this library's kernels launched in it.
Every decode step reads all weights (5.2 GB), far more than the 126 MB L2, so
no separate L2 flush is needed between iterations.

``--sizes 9b`` and ``--sizes 27b`` run the workloads named for those sizes: a batch of
8 prompts of unequal random lengths 512-4,096 and 256 decode steps; a batch of 16
prompts of 1,024-8,192 tokens and 128 decode steps (a prompt is at most as long as
leaves room for the decoded tokens in the context of 8192).  Their prefill figure is
the whole unequal batch in one step.  Bytes and flops of the rooflines are asked of
the model's parts (``Model.decode_bytes``, ``Model.prefill_flops``).
"""
from __future__ import annotations

import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent

# Gemma-2 2B layer sizes
GEMMA2_2B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 26, "hidden_size": 2304, "num_attention_heads": 8, "num_key_value_heads": 4,
    "head_dim": 256, "intermediate_size": 9216, "vocab_size": 256000, "rope_theta": 10000.0,
    "sliding_window": 4096, "query_pre_attn_scalar": 256, "attn_logit_softcapping": 50.0,
    "final_logit_softcapping": 30.0, "max_position_embeddings": 8192, "rms_norm_eps": 1e-6,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "torch_dtype": "bfloat16",
}
# the other sizes of the family differ in these keys (--sizes 9b / 27b: not the default run)
SIZES = {
    "2b": {},
    "9b": {"num_hidden_layers": 42, "hidden_size": 3584, "num_attention_heads": 16, "num_key_value_heads": 8,
           "intermediate_size": 14336},
    "27b": {"num_hidden_layers": 46, "hidden_size": 4608, "num_attention_heads": 32, "num_key_value_heads": 16,
            "head_dim": 128, "intermediate_size": 36864, "query_pre_attn_scalar": 144},
}
# what is run at each size: the batch, the prompts' lengths (one number: all equal; two: uniform random
# between them), the decode steps that are timed, and the batches of the extra decode points
WORKLOADS = {
    "2b": {"batch": 8, "prompt": (2048,), "steps": 256, "points": (1, 64)},
    "9b": {"batch": 8, "prompt": (512, 4096), "steps": 256, "points": ()},
    "27b": {"batch": 16, "prompt": (1024, 8192), "steps": 128, "points": ()},
}
PROMPT_LEN = 2048
CONTEXT = 8192
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.is_file():
        try:
            d = json.loads(p.read_text())
            return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]), "source": "measured"}
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def prefill_shares(prefill_once, model, lens, pk) -> dict:
    """The layers' products and the attention kernels of one prefill apart: the time charged to them
    (one more prefill under the CUDA profiler of PyTorch) and their flops over the bf16 peak."""
    import torch
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        prefill_once()
        torch.cuda.synchronize()
    # Kernels overlap (a kernel starts while the one in front still runs and waits for it): a kernel is
    # charged the time from the end of what ran before it to its own end, so that the shares add up to the
    # time the device was busy.
    evs = sorted((e for e in prof.events() if "cuda" in str(e.device_type).lower()), key=lambda e: e.time_range.start)
    gemm_us = attn_us = other_us = 0.0
    busy_until = None
    for e in evs:
        start, end = e.time_range.start, e.time_range.end
        own = end - start if busy_until is None else max(0.0, end - max(start, busy_until))
        busy_until = end if busy_until is None else max(busy_until, end)
        if "gemm_tc_kernel<256" in e.name or "gemm_tc_kernel<128" in e.name or "gemm_tc_pair_kernel" in e.name:
            gemm_us += own                                     # (the head's few rows are not among these)
        elif "attn_prefill" in e.name:
            attn_us += own
        else:
            other_us += own                                    # norms, rotary, embedding, head, copies
    attn = model.score_flops(lens)
    linear = model.prefill_flops(lens, 0) - attn
    peak = pk["bf16_tflops"] * 1e12
    out = {}
    if gemm_us > 0:
        out["products"] = {"ms": gemm_us / 1e3, "frac": linear / (gemm_us / 1e6) / peak}
    if attn_us > 0:
        out["attention"] = {"ms": attn_us / 1e3, "frac": attn / (attn_us / 1e6) / peak}
    out["other"] = {"ms": other_us / 1e3}
    return out


def run_ours(args) -> dict:
    import torch
    sys.path.insert(0, str(ROOT))
    from airframe_b200 import kernels, transfers
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine import GpuRuntime, StepEntry
    from airframe_b200.sampling import Sampler, SamplingParams

    work = dict(WORKLOADS[args.sizes])
    if args.prompt_len:
        work["prompt"] = (args.prompt_len,)
    B = args.batch or work["batch"]
    K = args.steps or work["steps"]
    W = max(args.warmup, 3)
    points = () if args.no_points else work["points"]
    full = dict(GEMMA2_2B, **SIZES[args.sizes])
    full_layers = full["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg_dict = dict(full, num_hidden_layers=n_layers)
    cfg = config_from_dict(cfg_dict)
    V = cfg.vocab_size
    pk = peaks()
    torch.manual_seed(0)
    room = CONTEXT - (K + max(W, 32) + 2)                      # a prompt leaves room for the tokens decoded after it

    def lengths(n, seed):
        spec = work["prompt"]
        if len(spec) == 1:
            return [min(spec[0], room)] * n
        g = torch.Generator().manual_seed(seed)
        hi = min(spec[1], room)
        return [int(x) for x in torch.randint(spec[0], hi + 1, (n,), generator=g)]

    def prompts(lens, seed):
        g = torch.Generator().manual_seed(seed)
        return [torch.randint(0, V, (n,), generator=g).tolist() for n in lens]

    def pages(n):
        return (n + K + W + 8 + 63) // 64 * 64

    main_lens = lengths(B, 100 + B)
    budget = max([sum(pages(n) for n in main_lens)] + [b * pages(min(PROMPT_LEN, room)) for b in points])
    max_b = max([B] + list(points))
    rt = GpuRuntime.random(cfg, seed=0, dtype="bfloat16", max_tokens=budget, max_context=CONTEXT,
                           max_sequences=max_b, on_device=True)
    eng = rt.engine
    model = eng.model
    dev = eng.device
    greedy = SamplingParams(max_tokens=1, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)

    def timed(fn, n):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(n):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end)

    def step_timeline(one):
        """Start and duration (us, device clock) of every kernel and copy of one decode step, as the
        CUDA profiler of PyTorch records them (the kernels of a graph replay overlap: a kernel's span
        includes its wait for the kernel in front)."""
        from torch.profiler import ProfilerActivity, profile
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            for _ in range(2):
                one()
            torch.cuda.synchronize()
        evs = sorted((e for e in prof.events() if "cuda" in str(e.device_type).lower()),
                     key=lambda e: e.time_range.start)
        first = [i for i, e in enumerate(evs) if "embed_kernel" in e.name][-1]
        t0 = evs[first].time_range.start
        return [(e.time_range.start - t0, e.time_range.end - e.time_range.start, e.name) for e in evs[first:]]

    def decode_rate(lens, steps, warm, clocks=None, timeline=None):
        """tokens/s, ms/step, launches and final lengths of `steps` decode steps of sequences whose prompts
        have `lens` tokens."""
        batch = len(lens)
        sampler = Sampler(V, dev)
        states = [sampler.new_state(greedy, i) for i in range(batch)]
        slots = [eng.take_slot() for _ in range(batch)]
        try:
            ps = prompts(lens, 100 + batch)
            first = eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, ps)], greedy=True)
            state = {}

            # the product's own way of stepping (GenerationLoop, greedy): a step gives its arg-max tokens (the
            # head's epilogue finds them; no logits are written), takes its input tokens from the device, where
            # the step before left them, and is queued before the host has read those
            state["pending"] = sampler.adopt(first, states)

            def one():
                toks = eng.decode_rows(slots, state["pending"].device, greedy=True)
                nxt = sampler.adopt(toks, states)
                state["pending"].result()                     # the tokens of the step before, on the host
                state["pending"] = nxt

            # The clocks, lowered by the burst of prompts, take some 30 steps to come back: the first decode step
            # (which captures the graph) is run SETTLE more times on the same inputs (the same rows into the
            # cache, the same tokens out), so that a short warm-up measures the same device as a long one.
            if warm > 0:
                one()
                eng.repeat_last_decode(SETTLE)
            for _ in range(max(warm - 1, 0)):
                one()
            if timeline is not None:
                timeline.extend(step_timeline(one))
            if clocks is not None:
                clocks.start()
            n0 = kernels.launch_count() + eng.replayed_launches
            ms = timed(one, steps)
            state["pending"].result()
            launches = kernels.launch_count() + eng.replayed_launches - n0
            after = [eng.length(s) for s in slots]
            return batch * steps / (ms / 1e3), ms / steps, launches, after
        finally:
            for s in slots:
                eng.free_slot(s)

    # ---- prefill: one 2,048-token sequence (the default run), or the workload's whole unequal batch in one step;
    #      logits at the last position of every sequence
    pf_lens = main_lens if len(work["prompt"]) > 1 else [main_lens[0]]
    pf_prompts = prompts(pf_lens, 7)

    def prefill_once():
        slots = [eng.take_slot() for _ in pf_prompts]
        try:
            eng.step([StepEntry(s, p, [len(p) - 1]) for s, p in zip(slots, pf_prompts)])
        finally:
            for s in slots:
                eng.free_slot(s)

    for _ in range(3):
        prefill_once()
    reps = 5
    pf_ms = timed(prefill_once, reps) / reps
    pf_tokens = sum(pf_lens)
    pf_flops = model.prefill_flops(pf_lens, len(pf_lens))
    prefill = {"value": pf_tokens / (pf_ms / 1e3), "tokens": pf_tokens, "ms": pf_ms,
               "frac": pf_flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12), "sequences": len(pf_lens)}

    if args.timeline:
        tl = []
        decode_rate(main_lens, 4, W, timeline=tl)
        print(f"# one decode step, batch {B}, {n_layers} layers: start us, duration us, kernel")
        for start, dur, name in tl:
            print(f"{start:9.1f} {dur:8.1f}  {name[:100]}")
        return None

    # ---- the headline: decode at batch B
    clocks = ClockSampler()
    value, ms_step, launches, after = decode_rate(main_lens, K, W, clocks)
    clock_info = clocks.stop()
    # the bytes a step has to read: every weight once and the cache of the live sequences, at the lengths they
    # have in the middle of the timed steps
    mid = [n - K // 2 for n in after]
    need = model.decode_bytes(mid)
    achieved = need / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"], "bytes": need}

    point_rates = {}
    for b in points:
        point_rates[f"decode_b{b}"] = decode_rate([min(PROMPT_LEN, room)] * b, max(4, K // 2), W)[0]

    # ---- end to end through the public entry point: We + K + 1 tokens a sequence, We = W but at least 32 (the
    #      generation loop cannot repeat a step: the clocks come back over its own first steps); the clock runs
    #      from the moment every sequence has its token We + 1 to the last token: K steps
    We = max(W, 32)
    n_new = We + K + 1
    stamps = []
    params = SamplingParams(max_tokens=n_new, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    ps = prompts(main_lens, 500)
    rt.generate(ps, SamplingParams(max_tokens=4, temperature=0.0, repetition_penalty=1.0, ignore_eos=True))
    moved = []

    def on_token(i, t):
        stamps.append(time.perf_counter())
        if len(stamps) == (We + 1) * B:           # the warm-up steps are done
            moved.append(transfers.snapshot())

    rt.generate(ps, params, on_token=on_token)
    torch.cuda.synchronize()
    moved.append(transfers.snapshot())
    t_first = stamps[(We + 1) * B - 1]
    e2e_value = B * K / (stamps[-1] - t_first)
    # bytes counted where they are copied (token ids, positions, slots, lengths and page-table rows in;
    # sampled tokens out), over the decode steps of the timed run
    e2e = {"value": e2e_value, "unit": "tokens/s",
           "h2d_bytes_per_step": round((moved[1][0] - moved[0][0]) / K),
           "d2h_bytes_per_step": round((moved[1][1] - moved[0][1]) / K)}

    # (last, so that the launches before it come in the same order with and without it)
    try:
        prefill["profiled"] = dict(prefill_shares(prefill_once, model, pf_lens, pk),
                                   note="kernel times of one more prefill under the CUDA profiler of PyTorch, "
                                        "not timed with events like the figures beside it")
    except Exception as why:        # a profiler that cannot attach (another one is attached already) costs only this key
        prefill["profiled"] = {"unavailable": str(why)[:120]}

    equal = len(work["prompt"]) == 1
    what = f"{main_lens[0]:,}-token prompts" if equal else f"prompts of {work['prompt'][0]:,}-{min(work['prompt'][1], room):,} tokens"
    return {
        "metric": f"Gemma-2 {args.sizes.upper()} bf16 decode tokens/s at batch {B} ({what})",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), uniform random token ids",
        "config": {"model": f"gemma-2-{args.sizes} sizes", "global_batch": B,
                   "seq_len": main_lens[0] if equal else round(sum(main_lens) / B), "context": CONTEXT,
                   "prompt_lens": "equal" if equal else f"uniform random, mean {round(sum(main_lens) / B)}, "
                                                         f"min {min(main_lens)}, max {max(main_lens)}",
                   "parallelism": "single-gpu", "layers": n_layers, "layers_full": full_layers,
                   "hidden": cfg_dict["hidden_size"], "heads": cfg_dict["num_attention_heads"],
                   "kv_heads": cfg_dict["num_key_value_heads"], "head_dim": cfg_dict["head_dim"],
                   "intermediate": cfg_dict["intermediate_size"], "vocab": cfg_dict["vocab_size"],
                   "sliding_window": cfg_dict["sliding_window"], "sampling": "greedy, in the head's epilogue",
                   "l2": f"inputs larger than L2 (weights {model.decode_bytes([]) / 1e9:.1f} GB per step)",
                   "settle": f"{SETTLE} untimed replays of the first decode step on its own inputs before the warm-up"},
        "prefill": prefill, "roofline": roofline, "points": point_rates, "e2e": e2e,
        "gpu_launches": launches, "clocks": clock_info, "impl": "ours",
    }


SETTLE = 64     # replays of the first decode step on its own inputs before the warm-up steps go on


def attention_points() -> None:
    """The decode attention kernels alone (split + merge, the cut from a step's plan) at the shapes of the three
    sizes' workloads: a CUDA graph of 12 launches back to back over caches larger than L2, taken in turn; CUDA events."""
    import torch
    from airframe_b200 import kernels as K
    dev, page = torch.device("cuda:0"), 64

    def case(tag, nq, nkv, hd, lens, n_caches):
        B = len(lens)
        per = max((n + page - 1) // page for n in lens)
        n_pages = B * per
        caches = [(torch.randn(n_pages, nkv, page, hd, device=dev).bfloat16(),
                   torch.randn(n_pages, nkv, page, hd, device=dev).bfloat16()) for _ in range(n_caches)]
        table = torch.randperm(n_pages, device=dev).int().reshape(B, per).contiguous()
        slots = torch.arange(B, device=dev, dtype=torch.int32)
        lens_t = torch.tensor(lens, device=dev, dtype=torch.int32)
        q = torch.randn(B, nq * hd, device=dev).bfloat16()
        out = torch.empty_like(q)
        nbytes = sum((n + page - 1) // page for n in lens) * page * nkv * hd * 2 * 2
        n = K.attn_decode_max_splits(B, nkv, max(lens), 0, nq=nq)
        scratch = torch.empty(B * nq * n * (hd + 2), device=dev)
        plan = K.attn_decode_plan(table, slots, lens_t, nq, nkv, 0, 0, n)

        def run(i):
            kc, vc = caches[i % n_caches]
            K.attn_decode_split(out, q, kc, vc, table, slots, lens_t, nq, nkv, hd, hd ** -0.5, 50.0, 0, 0, n,
                                scratch, plan=plan)
        for i in range(3):
            run(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(12):
                run(i)
        graph.replay()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(10):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / 120 * 1000
        print(f"{tag:44s} {us:8.2f} us a launch  {nbytes / us / 1e6:6.2f} TB/s  ({nbytes / 1e6:.0f} MB of cache pages)",
              flush=True)

    case("2b sizes, 8 x 2,049 tokens", 8, 4, 256, [2049] * 8, 6)
    case("2b sizes, 1 x 2,049", 8, 4, 256, [2049], 16)
    case("2b sizes, 64 x 2,049", 8, 4, 256, [2049] * 64, 2)
    case("2b sizes, 32 short ones of 100 ... 410", 8, 4, 256, [100 + 10 * i for i in range(32)], 8)
    case("2b sizes, one of 8,000 among 15 of 300", 8, 4, 256, [300] * 15 + [8000], 4)
    case("9b sizes, 8 of 512 ... 4,096", 16, 8, 256, [512 * (i + 1) for i in range(8)], 3)
    case("9b sizes, 8 x 2,304 (the same bytes)", 16, 8, 256, [2304] * 8, 3)
    case("27b sizes, 16 of 1,024 ... 8,194", 32, 16, 128, [1024 + i * 478 for i in range(16)], 2)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=0, help="decode steps that are timed (default: the workload's, 256 at 2b)")
    ap.add_argument("--warmup", type=int, default=32,
                    help="untimed decode steps after the prompts (the first 30 or so after a burst of prompts "
                         "run at lowered clocks)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=0, help="sequences of the decode batch (default: the workload's, 8 at 2b)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels of one decode step with their start and duration, then exit")
    ap.add_argument("--prompt-len", type=int, default=0,
                    help="equal prompts of this many tokens instead of the workload's (not the default run)")
    ap.add_argument("--attention", action="store_true",
                    help="time the decode attention kernels alone at the workloads' shapes, then exit")
    ap.add_argument("--sizes", default="2b", choices=sorted(SIZES),
                    help="layer sizes of this Gemma-2 model, with the workload named for them")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate on wgpu (no setup.py/pyproject.toml: pip cannot install "
                          "it; no Rust toolchain; no graphics stack on this box)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.attention:
        attention_points()
        return 0
    line = run_ours(args)
    if line is not None:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
