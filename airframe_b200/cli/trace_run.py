"""``trace_run``: feed given token ids through a model step by step and write
logits.  It samples nothing and has no forward pass, cache or loader of its
own: it drives :class:`~airframe_b200.engine.GpuRuntime`'s step function.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come on standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

The requests of a step either all start or all go on by one token.  For a step
in which something is wanted, ``DIR/<step>.f32`` receives the logits at the
wanted places, in the order of the entries and of ``want``, as little-endian
32-bit floats [wanted, vocab].  After every step a line ``done <step>`` is
printed and flushed.  Requests named in ``end`` give back what they hold.
With ``--layers``, a step in which something is wanted also writes
``DIR/<step>.layers.json``: per scheduled run of a layer, for every wanted row of
the residual stream, its RMS, first 20 values and bit-sum checksum (the
localizer of :mod:`airframe_b200.engine.probe`; such steps run kernel by kernel).

Reference: the fixture-driven replays (``src/runtime/multi_token_engine.rs:199-205``,
``src/bin/invariant_probe.rs:1-20``) and the one-token-at-a-time trace of
``src/bin/shimmy_server_gpu/server_inference.rs:778-926``.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path


def main(argv=None, stdin=None, stdout=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description="replay token ids step by step, write logits")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--layers", action="store_true",
                    help="also write <step>.layers.json: per layer RMS, first values and checksum of the wanted rows")
    args = ap.parse_args(argv)
    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout

    import torch
    from .. import kernels
    from ..config import config_from_folder
    from ..engine import GpuRuntime, LayerProbe, StepEntry

    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    limit = config_from_folder(args.model).model_spec().max_positions
    rt = GpuRuntime.load(args.model, dtype=args.dtype, device=args.device, max_tokens=args.max_tokens,
                         max_context=limit)
    slots: dict = {}
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        taken = []
        try:
            for e in rec.get("entries", []):
                rid = e["id"]
                if rid not in slots:
                    slots[rid] = rt.engine.take_slot()
                    taken.append(rid)
                entries.append(StepEntry(slots[rid], [int(t) for t in e["tokens"]],
                                         [int(w) for w in e.get("want", [])]))
            if entries:
                probe = LayerProbe() if args.layers and any(e.want for e in entries) else None
                logits = rt.step(entries, probe=probe)
                if probe is not None:
                    tmp = out_dir / f"{step}.layers.json.tmp"
                    tmp.write_text(json.dumps(probe.to_json()))
                    tmp.replace(out_dir / f"{step}.layers.json")
                if logits is not None:
                    data = logits.to(torch.float32).contiguous().cpu().numpy().astype("<f4", copy=False)
                    tmp = out_dir / f"{step}.f32.tmp"
                    data.tofile(tmp)
                    tmp.replace(out_dir / f"{step}.f32")
                else:
                    torch.cuda.synchronize()
                kernels.check_device_errors(rt.engine.device)     # a kernel that gave up waiting fails the step
        except Exception:
            for rid in taken:
                rt.engine.free_slot(slots.pop(rid))
            raise
        for rid in rec.get("end", []):
            if rid in slots:
                rt.engine.free_slot(slots.pop(rid))
        print(f"done {step}", file=stdout, flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
