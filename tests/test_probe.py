"""The per-layer localizer: its facts on the CPU, and on the GPU that the facts
of the engine's residual stream agree with the plain implementation layer by
layer and that a fault planted in one layer is named as that layer."""
import json
import shutil
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_gemma2 as plain
import replay
from tiny import CONFIGS, make_folder

ROOT = Path(__file__).resolve().parent.parent


def test_row_facts_are_what_they_say():
    from airframe_b200.engine.probe import first_difference, row_facts
    row = np.array([1.0, -2.0, 0.5, 3.0], dtype=np.float32)
    f = row_facts(row, first=3)
    assert f["rms"] == pytest.approx(float(np.sqrt((1 + 4 + 0.25 + 9) / 4)))
    assert f["first"] == [1.0, -2.0, 0.5]
    # the bit patterns of the floats, added as 64-bit integers: a changed bit anywhere changes it
    want = sum(int(np.float32(v).view(np.uint32)) for v in row)
    assert f["checksum"] == want
    row2 = row.copy()
    row2[3] = np.nextafter(row2[3], np.float32(4.0))
    assert row_facts(row2)["checksum"] == want + 1
    ref = [[[1.0, 1.0]], [[2.0, -2.0]], [[3.0, 3.0]]]                      # [run][row] -> the other implementation's row
    recs = [{"run": -1, "layer": -1, "rows": [{"rms": 9.0, "first": [9.0]}]},
            {"run": 0, "layer": 0, "rows": [{"rms": 1.0, "first": [1.0, 1.0]}]},
            {"run": 1, "layer": 1, "rows": [{"rms": 2.0, "first": [2.0, 2.0]}]},    # the same size, another direction
            {"run": 2, "layer": 2, "rows": [{"rms": 9.0, "first": [3.0, 3.0]}]}]
    assert first_difference(recs, ref, 0.05) == (1, 1, 0)
    assert first_difference(recs[:2], ref, 0.05) is None
    recs[2]["rows"][0]["first"] = [2.0, -2.0]
    assert first_difference(recs, ref, 0.05) == (2, 2, 0)                  # now only the size of run 2 is off


def _plain_facts(cfg, w, ids, rows):
    out = []
    for k in range(cfg["num_hidden_layers"]):
        x = plain.hidden_states(cfg, w, ids, upto_layer=k + 1)
        out.append([x[r] for r in rows])
    return out


@pytest.mark.gpu
@pytest.mark.parametrize("dtype,tol", [("float32", 1e-4), ("bfloat16", 3e-2)])
def test_layers_agree_with_the_plain_implementation_and_a_fault_is_named(dtype, tol, tmp_path):
    from airframe_b200.engine import GpuRuntime, LayerProbe, StepEntry
    from airframe_b200.weights.safetensors_io import write_safetensors
    name = "C"
    folder = make_folder(CONFIGS[name], seed=3, store_dtype="bfloat16", root=tmp_path / "good")
    cfg, w = plain.read_model_folder(folder)
    ids = replay.random_ids(cfg["vocab_size"], 90, 5)
    rows = [0, 41, 89]
    ref = _plain_facts(cfg, w, ids, rows)
    ref_rms = [[float(r.pow(2).mean().sqrt()) for r in layer] for layer in ref]
    ref_rows = [[r.tolist() for r in layer] for layer in ref]

    def probed(path):
        rt = GpuRuntime.load(path, dtype=dtype, max_tokens=256)
        s = rt.engine.take_slot()
        try:
            probe = LayerProbe()
            rt.step([StepEntry(s, ids, rows)], probe=probe)
            return probe.records
        finally:
            rt.engine.free_slot(s)

    from airframe_b200.engine.probe import first_difference
    recs = probed(folder)
    assert [r["run"] for r in recs] == [-1, 0, 1, 2, 3] and [r["layer"] for r in recs] == [-1, 0, 1, 2, 3]
    for rec in recs[1:]:
        for r, facts in enumerate(rec["rows"]):
            want = ref[rec["run"]][r]
            assert facts["rms"] == pytest.approx(ref_rms[rec["run"]][r], rel=tol)
            got = torch.tensor(facts["first"], dtype=torch.float64)
            assert float((got - want[:20]).abs().max()) <= tol * float(want.abs().max())
    assert first_difference(recs, ref_rows, tol) is None
    # a fault in layer 2 (half of its down projection's rows three times too large; all of them would be
    # undone by the norm that follows): the first run that differs is run 2
    bad = tmp_path / "bad"
    shutil.copytree(folder, bad)
    tensors = plain.read_safetensors(bad / "model.safetensors")
    key = "model.layers.2.mlp.down_proj.weight"
    wrong = tensors[key].float()
    wrong[: wrong.shape[0] // 2] *= 3.0
    tensors[key] = wrong.to(tensors[key].dtype)
    write_safetensors(bad / "model.safetensors",
                      [(n, tuple(t.shape), t.dtype, (lambda t=t: t)) for n, t in tensors.items()])
    assert first_difference(probed(bad), ref_rows, tol)[:2] == (2, 2)


@pytest.mark.gpu
def test_trace_run_writes_layer_facts(tmp_path):
    folder = make_folder(CONFIGS["A"], seed=4, store_dtype="bfloat16", root=tmp_path / "model")
    cfg, w = plain.read_model_folder(folder)
    ids = replay.random_ids(cfg["vocab_size"], 12, 9)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": ids[:11], "want": [10]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": ids[11:], "want": [0]}], "end": ["a"]}]
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", "float32",
                           "--out", str(out), "--max-tokens", "64", "--layers"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    ref = plain.hidden_states(cfg, w, ids)
    for step, pos in ((0, 10), (1, 11)):
        recs = json.loads((out / f"{step}.layers.json").read_text())
        last = recs[-1]
        assert last["layer"] == cfg["num_hidden_layers"] - 1 and len(last["rows"]) == 1
        assert last["rows"][0]["rms"] == pytest.approx(float(ref[pos].pow(2).mean().sqrt()), rel=1e-4)
        assert (out / f"{step}.f32").exists()
