"""bin/trace_run as a user runs it: a subprocess fed steps on standard input."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gemma2 as plain
import replay
from tiny import CONFIGS, make_folder
from tolerances import SPLITS, VS_PLAIN, rel_err

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run_trace(folder, dtype, steps, out_dir, max_tokens):
    text = "".join(json.dumps(s) + "\n" for s in steps)
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
                           "--out", str(out_dir), "--max-tokens", str(max_tokens)], input=text,
                          capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert proc.stdout.split() == [w for s in steps for w in ("done", str(s["step"]))]
    return proc


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("B", "bfloat16"), ("C", "bfloat16"), ("A", "float32")])
def test_replay_whole_tail_and_batches(name, dtype, tmp_path):
    folder = make_folder(CONFIGS[name], seed=31, store_dtype="bfloat16", root=tmp_path / "model")
    cfg, w = plain.read_model_folder(folder)
    V = cfg["vocab_size"]
    lens = {"A": [40, 64, 7], "B": [70, 128, 33], "C": [150, 40, 260]}[name]
    reqs = {f"r{i}": replay.random_ids(V, n, 300 + i) for i, n in enumerate(lens)}
    ref = {k: plain.logits(cfg, w, v) for k, v in reqs.items()}
    steps, where = [], []          # where: (step, request, first position, count)
    n = 0
    # 1. each request alone and whole
    for k, ids in reqs.items():
        steps.append({"step": n, "entries": [{"id": k + "w", "tokens": ids, "want": list(range(len(ids)))}],
                      "end": [k + "w"]})
        where.append((n, [(k, 0, len(ids))], "whole"))
        n += 1
    # 2. the last 32 tokens one by one
    for k, ids in reqs.items():
        head = max(1, len(ids) - 32)
        steps.append({"step": n, "entries": [{"id": k + "t", "tokens": ids[:head], "want": [head - 1]}], "end": []})
        where.append((n, [(k, head - 1, 1)], "tail"))
        n += 1
        for p in range(head, len(ids)):
            steps.append({"step": n, "entries": [{"id": k + "t", "tokens": [ids[p]], "want": [0]}],
                          "end": [k + "t"] if p == len(ids) - 1 else []})
            where.append((n, [(k, p, 1)], "tail"))
            n += 1
    # 3. a batch of unequal prompts, one token each afterwards, shorter requests end earlier; twice,
    #    so that the second batch gets the slots and pages of the first
    for rnd in range(2):
        fed = {k: max(1, len(ids) // 3) for k, ids in reqs.items()}
        steps.append({"step": n, "entries": [{"id": f"{k}b{rnd}", "tokens": reqs[k][:fed[k]], "want": [fed[k] - 1]}
                                             for k in reqs], "end": []})
        where.append((n, [(k, fed[k] - 1, 1) for k in reqs], "batch"))
        n += 1
        live = list(reqs)
        while live:
            ending = [k for k in live if fed[k] + 1 >= len(reqs[k])]
            steps.append({"step": n, "entries": [{"id": f"{k}b{rnd}", "tokens": [reqs[k][fed[k]]], "want": [0]}
                                                 for k in live], "end": [f"{k}b{rnd}" for k in ending]})
            where.append((n, [(k, fed[k], 1) for k in live], "batch"))
            for k in live:
                fed[k] += 1
            live = [k for k in live if k not in ending]
            n += 1
    # a step in which nothing is wanted writes no file
    steps.append({"step": n, "entries": [{"id": "quiet", "tokens": [1, 2, 3], "want": []}], "end": ["quiet"]})
    quiet = n
    budget = sum((len(v) + 63) // 64 * 64 for v in reqs.values())       # all three live at once, no more
    out_dir = tmp_path / "out"
    run_trace(folder, dtype, steps, out_dir, budget)
    assert not (out_dir / f"{quiet}.f32").exists()
    whole = {}
    for step, parts, kind in where:
        data = torch.from_numpy(np.fromfile(out_dir / f"{step}.f32", dtype="<f4").reshape(-1, V).copy())
        assert data.shape[0] == sum(c for _, _, c in parts)
        o = 0
        for k, first, count in parts:
            got = data[o:o + count]
            o += count
            assert rel_err(got, ref[k][first:first + count]) < VS_PLAIN[dtype], (step, kind, k, first)
            if kind == "whole":
                whole[k] = got
            else:
                assert rel_err(got, whole[k][first:first + count]) < SPLITS[dtype], (step, kind, k, first)


def test_replay_refuses_more_tokens_than_it_was_sized_for(tmp_path):
    folder = make_folder(CONFIGS["B"], seed=1, root=tmp_path / "model")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": list(range(65)), "want": []},
                                     {"id": "b", "tokens": [1], "want": []}], "end": []}]
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype",
                           "float32", "--out", str(tmp_path / "o"), "--max-tokens", "128"],
                          input=json.dumps(steps[0]) + "\n", capture_output=True, text=True, timeout=900)
    assert proc.returncode != 0 and "CacheFull" in proc.stderr
