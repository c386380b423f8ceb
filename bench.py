#!/usr/bin/env python3
"""Decode and prefill throughput of Gemma-2 2B sizes (random weights, bf16) on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

A step is one decode step of a batch of 8 sequences that hold 2,048-token
prompts (context limit 8192): the model's step function plus greedy sampling on
the device, stepped as the generation loop steps it (a step takes its tokens from
the device and is queued before the host has read them).  ``value`` is decoded
tokens a second, timed with CUDA events around exactly K steps after W warm-up
steps (default 32: the first 30 or so steps after a burst of prompts run at
lowered clocks, about 2.1 ms instead of 1.8).  ``e2e`` is the same through
``GpuRuntime.generate`` with host token lists in and out, prompts' aftermath included.  The line also carries
the prefill rate of 2,048 tokens with its fraction of the bf16 peak (and, under ``profiled``,
the same for its products and its attention kernels apart, from a run under a profiler), the decode
step's fraction of the HBM roofline, decode at batch 1 and 64, the clocks seen
during the timed region and the number of this library's kernels launched in it.
Every decode step reads all weights (5.2 GB), far more than the 126 MB L2, so
no separate L2 flush is needed between iterations.
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


def model_bytes(cfg, n_layers):
    """Bytes of the weights a decode step reads once (bf16)."""
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    per_layer = (q + 2 * kv) * h + h * q + 3 * h * i + 4 * h
    return 2 * (n_layers * per_layer + v * h + h)


def cache_bytes(cfg, n_layers, lens):
    """Bytes of keys and values a decode step reads for sequences of these lengths."""
    kv_row = 2 * cfg["num_key_value_heads"] * cfg["head_dim"] * 2
    total = 0
    for layer in range(n_layers):
        sliding = layer % 2 == 0
        for n in lens:
            total += kv_row * (min(n, cfg["sliding_window"]) if sliding else n)
    return total


def prefill_flops(cfg, n_layers, T, n_logits):
    h, i, v = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2 * T * n_layers * ((q + 2 * kv) * h + h * q + 3 * h * i)
    attn = 0
    for layer in range(n_layers):
        w = cfg["sliding_window"] if layer % 2 == 0 else None
        pairs = sum(min(t + 1, w) if w else t + 1 for t in range(T))
        attn += 2 * 2 * pairs * q
    return linear + attn + 2 * n_logits * v * h


def prefill_shares(prefill_once, cfg, n_layers, pk) -> dict:
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
    gemm_us = attn_us = 0.0
    busy_until = None
    for e in evs:
        start, end = e.time_range.start, e.time_range.end
        own = end - start if busy_until is None else max(0.0, end - max(start, busy_until))
        busy_until = end if busy_until is None else max(busy_until, end)
        if "gemm_tc_kernel<256" in e.name or "gemm_tc_kernel<128" in e.name:     # (the head's one row is not among these)
            gemm_us += own
        elif "attn_prefill" in e.name:
            attn_us += own
    h, i = cfg["hidden_size"], cfg["intermediate_size"]
    q = cfg["num_attention_heads"] * cfg["head_dim"]
    kv = cfg["num_key_value_heads"] * cfg["head_dim"]
    linear = 2 * PROMPT_LEN * n_layers * ((q + 2 * kv) * h + h * q + 3 * h * i)
    attn = prefill_flops(cfg, n_layers, PROMPT_LEN, 0) - linear
    peak = pk["bf16_tflops"] * 1e12
    out = {}
    if gemm_us > 0:
        out["products"] = {"ms": gemm_us / 1e3, "frac": linear / (gemm_us / 1e6) / peak}
    if attn_us > 0:
        out["attention"] = {"ms": attn_us / 1e3, "frac": attn / (attn_us / 1e6) / peak}
    return out


def run_ours(args) -> dict:
    global PROMPT_LEN
    PROMPT_LEN = args.prompt_len
    import torch
    sys.path.insert(0, str(ROOT))
    from airframe_b200 import kernels
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine import GpuRuntime, StepEntry
    from airframe_b200.sampling import Sampler, SamplingParams

    full = dict(GEMMA2_2B, **SIZES[args.sizes])
    full_layers = full["num_hidden_layers"]
    n_layers = args.layers or full_layers
    cfg_dict = dict(full, num_hidden_layers=n_layers)
    cfg = config_from_dict(cfg_dict)
    B, K, W = args.batch, args.steps, max(args.warmup, 3)
    pk = peaks()
    torch.manual_seed(0)
    max_b = max([B] + ([] if args.no_points else [1, 64]))
    budget = max_b * ((PROMPT_LEN + K + W + 8 + 63) // 64 * 64)
    rt = GpuRuntime.random(cfg, seed=0, dtype="bfloat16", max_tokens=budget, max_context=CONTEXT,
                           max_sequences=max_b, on_device=True)
    eng = rt.engine
    dev = eng.device
    V = cfg.vocab_size
    greedy = SamplingParams(max_tokens=1, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)

    def prompts(n, seed):
        g = torch.Generator().manual_seed(seed)
        return [torch.randint(0, V, (PROMPT_LEN,), generator=g).tolist() for _ in range(n)]

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

    def decode_rate(batch, steps, warm, clocks=None, timeline=None):
        """tokens/s, ms/step and launches of `steps` decode steps at `batch` after 2,048-token prompts."""
        sampler = Sampler(V, dev)
        states = [sampler.new_state(greedy, i) for i in range(batch)]
        slots = [eng.take_slot() for _ in range(batch)]
        try:
            ps = prompts(batch, 100 + batch)
            first = eng.step([StepEntry(s, p, [PROMPT_LEN - 1]) for s, p in zip(slots, ps)], greedy=True)
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

            for _ in range(warm):
                one()
            if timeline is not None:
                timeline.extend(step_timeline(one))
            if clocks is not None:
                clocks.start()
            n0 = kernels.launch_count() + eng.replayed_launches
            ms = timed(one, steps)
            state["pending"].result()
            launches = kernels.launch_count() + eng.replayed_launches - n0
            lens = [eng.length(s) for s in slots]
            return batch * steps / (ms / 1e3), ms / steps, launches, lens
        finally:
            for s in slots:
                eng.free_slot(s)

    # ---- prefill of 2,048 tokens (one sequence, logits at its last position)
    def prefill_once():
        s = eng.take_slot()
        try:
            eng.step([StepEntry(s, pf_prompt, [PROMPT_LEN - 1])])
        finally:
            eng.free_slot(s)

    pf_prompt = prompts(1, 7)[0]
    for _ in range(3):
        prefill_once()
    reps = 5
    pf_ms = timed(prefill_once, reps) / reps
    pf_flops = prefill_flops(cfg_dict, n_layers, PROMPT_LEN, 1)
    prefill = {"value": PROMPT_LEN / (pf_ms / 1e3), "tokens": PROMPT_LEN, "ms": pf_ms,
               "frac": pf_flops / (pf_ms / 1e3) / (pk["bf16_tflops"] * 1e12)}

    if args.timeline:
        tl = []
        decode_rate(B, 4, W, timeline=tl)
        print(f"# one decode step, batch {B}, {n_layers} layers: start us, duration us, kernel")
        for start, dur, name in tl:
            print(f"{start:9.1f} {dur:8.1f}  {name[:100]}")
        return None

    # ---- the headline: decode at batch B
    clocks = ClockSampler()
    value, ms_step, launches, lens = decode_rate(B, K, W, clocks)
    clock_info = clocks.stop()
    need = model_bytes(cfg_dict, n_layers) + cache_bytes(cfg_dict, n_layers, lens)
    achieved = need / (ms_step / 1e3) / 1e9
    roofline = {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": achieved / pk["hbm_gbs"], "peaks": pk["source"]}

    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = decode_rate(b, max(4, K // 2), W)[0]

    # ---- end to end through the public entry point
    n_new = K + 1
    stamps = []
    params = SamplingParams(max_tokens=n_new, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    ps = prompts(B, 500)
    rt.generate(ps, SamplingParams(max_tokens=4, temperature=0.0, repetition_penalty=1.0, ignore_eos=True))
    from airframe_b200 import transfers
    moved = []

    def on_token(i, t):
        stamps.append(time.perf_counter())
        if len(stamps) == B:                      # every sequence has its first token: the prompts are done
            moved.append(transfers.snapshot())

    rt.generate(ps, params, on_token=on_token)
    torch.cuda.synchronize()
    moved.append(transfers.snapshot())
    t_first = stamps[B - 1]
    e2e_value = B * (n_new - 1) / (stamps[-1] - t_first)
    # bytes counted where they are copied (token ids, positions, slots, lengths and page-table rows in;
    # sampled tokens out), over the decode steps of the timed run
    e2e = {"value": e2e_value, "unit": "tokens/s",
           "h2d_bytes_per_step": round((moved[1][0] - moved[0][0]) / (n_new - 1)),
           "d2h_bytes_per_step": round((moved[1][1] - moved[0][1]) / (n_new - 1))}

    # (last, so that the launches before it come in the same order with and without it)
    try:
        prefill["profiled"] = dict(prefill_shares(prefill_once, cfg_dict, n_layers, pk),
                                   note="kernel times of one more prefill under the CUDA profiler of PyTorch, "
                                        "not timed with events like the figures beside it")
    except Exception as why:        # a profiler that cannot attach (another one is attached already) costs only this key
        prefill["profiled"] = {"unavailable": str(why)[:120]}

    return {
        "metric": f"Gemma-2 {args.sizes.upper()} bf16 decode tokens/s at batch {B} ({PROMPT_LEN:,}-token prompts)",
        "value": value, "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W, "ms_per_step": ms_step,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights N(0, 0.02), uniform random token ids",
        "config": {"model": f"gemma-2-{args.sizes} sizes", "global_batch": B, "seq_len": PROMPT_LEN, "context": CONTEXT,
                   "parallelism": "single-gpu", "layers": n_layers, "layers_full": full_layers,
                   "hidden": cfg_dict["hidden_size"], "heads": cfg_dict["num_attention_heads"],
                   "kv_heads": cfg_dict["num_key_value_heads"], "head_dim": cfg_dict["head_dim"],
                   "intermediate": cfg_dict["intermediate_size"], "vocab": cfg_dict["vocab_size"],
                   "sliding_window": cfg_dict["sliding_window"], "sampling": "greedy, in the head's epilogue",
                   "l2": f"inputs larger than L2 (weights {model_bytes(cfg_dict, n_layers) / 1e9:.1f} GB per step)"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
        "gpu_launches": launches, "clocks": clock_info, "impl": "ours",
    }


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=32,
                    help="untimed decode steps after the prompts (the first 30 or so after a burst of prompts "
                         "run at lowered clocks)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    ap.add_argument("--no-points", action="store_true", help="skip decode at batch 1 and 64")
    ap.add_argument("--timeline", action="store_true",
                    help="print the kernels of one decode step with their start and duration, then exit")
    ap.add_argument("--prompt-len", type=int, default=PROMPT_LEN,
                    help="tokens of every prompt, and of the prefill that is timed (not the default run)")
    ap.add_argument("--sizes", default="2b", choices=sorted(SIZES), help="layer sizes of this Gemma-2 model")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a Rust crate on wgpu (no setup.py/pyproject.toml: pip cannot install "
                          "it; no Rust toolchain; no graphics stack on this box)"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    line = run_ours(args)
    if line is not None:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
