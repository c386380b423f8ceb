"""``simple_flight``: load a model folder, generate from token-id prompts,
print the new ids.  In the manner of the reference's example
(``examples/simple_flight.rs:12-69``): the model comes from ``--model`` or the
``LIBSHIMMY_MODEL_PATH`` variable, the prompt is positional, 32 greedy tokens
by default, generation stops at the end token, and it closes with "Flight
Complete".  Prompts are token ids ("5,17,3"), positional or after
``--prompt-ids``; several prompts make a batch.  ``--random NAME`` runs a named
configuration with seeded random weights instead of a folder.
Sampling options carry the names of ``SamplingParams``
(``src/runtime/gpu.rs:25-47``).
"""
from __future__ import annotations

import argparse
import os
import sys
import time


def parse_ids(text: str) -> list:
    try:
        ids = [int(t) for t in text.replace(",", " ").split()]
    except ValueError:
        raise SystemExit(f"simple_flight: a prompt is a list of token ids, got {text!r}")
    if not ids:
        raise SystemExit("simple_flight: a prompt needs at least one token id")
    return ids


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="simple_flight", description=__doc__.split("\n\n")[0])
    ap.add_argument("prompt", nargs="*", help='token ids of one request, e.g. "2,17,3"; repeat for a batch')
    ap.add_argument("--model", default=os.environ.get("LIBSHIMMY_MODEL_PATH"),
                    help="model folder (config.json, model.safetensors); default $LIBSHIMMY_MODEL_PATH")
    ap.add_argument("--random", metavar="NAME", default=None,
                    help="no folder: seeded random weights of a named configuration (tinyA, tinyB, 2b, 9b, 27b)")
    ap.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                    help="token ids of one request (as the positional prompts); may be repeated")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"])
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy (the example's sampler)")
    ap.add_argument("--top-p", type=float, default=0.95)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--stop-token-id", type=int, action="append", default=[])
    ap.add_argument("--ignore-eos", action="store_true")
    ap.add_argument("--max-context", type=int, default=None)
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)
    if not args.model and not args.random:
        ap.error("no model: give --model DIR, --random NAME, or set LIBSHIMMY_MODEL_PATH")
    prompts = [parse_ids(p) for p in list(args.prompt) + list(args.prompt_ids)] or [[2]]
    dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(args.dtype, args.dtype)

    from ..engine import GpuRuntime
    from ..sampling import SamplingParams

    print("SIMPLE FLIGHT CHECK")
    print("-------------------")
    print(f"Model: {args.random + ' (random weights, seed ' + str(args.seed) + ')' if args.random else args.model}")
    for p in prompts:
        print(f"Tokens: {p}")
    print("Loading airframe_b200...")
    need = sum((len(p) + args.max_tokens + 63) // 64 * 64 for p in prompts)
    if args.random:
        from ..config import config_from_dict
        from ..config.presets import preset
        try:
            cfg = config_from_dict(preset(args.random))
        except KeyError as e:
            ap.error(str(e.args[0]))
        rt = GpuRuntime.random(cfg, seed=args.seed, dtype=dtype, device=args.device, max_tokens=need,
                               max_context=args.max_context, on_device=True)
    else:
        rt = GpuRuntime.load(args.model, dtype=dtype, device=args.device, max_tokens=need,
                             max_context=args.max_context)
    print(f"Weights loaded: {len(rt.model.weight_decls())}")
    params = SamplingParams(max_tokens=args.max_tokens, temperature=args.temperature, top_p=args.top_p,
                            repetition_penalty=args.repetition_penalty, seed=args.seed,
                            stop_token_ids=list(args.stop_token_id), ignore_eos=args.ignore_eos)
    single = len(prompts) == 1

    def on_token(index, token):
        if single:
            print(token, end=" ", flush=True)

    if single:
        print("\nOutput: ", end="", flush=True)
    t0 = time.time()
    outs = rt.generate(prompts, params, on_token)
    dt = time.time() - t0
    if single:
        print()
    else:
        for i, o in enumerate(outs):
            print(f"Output {i}: {' '.join(map(str, o))}")
    n = sum(len(o) for o in outs)
    print(f"\n{n} tokens in {dt:.3f} s ({n / dt if dt > 0 else 0:.1f} tok/s)")
    print("\nFlight Complete.")
    return 0


if __name__ == "__main__":
    sys.exit(main())
