"""The checked build of the kernel library (``-DAF_BOUNDS_CHECK``): the indices that kernels take from data
are checked, a bad one is recorded and its access skipped.  Run in a process of its own (the build is chosen
before the library's first use): a tiny model's requests, cut in every way, touch no bad index and give the
plain logits; a page-table entry that was never assigned is recorded, and nothing is written for it."""
import subprocess
import sys
import textwrap
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

SCRIPT = textwrap.dedent('''
    import sys
    sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
    import torch
    import airframe_b200.csrc as csrc
    csrc.use_checked_build()
    from airframe_b200 import kernels as K
    assert K.bounds_failures() == (0, 0), "the checked build answers with a record"
    import plain_gemma2 as plain, replay
    from tiny import CONFIGS, make_folder
    from tolerances import VS_PLAIN, rel_err
    from airframe_b200.engine import GpuRuntime
    for name, dtype in (("A", "float32"), ("B", "bfloat16"), ("H", "bfloat16")):
        folder = make_folder(CONFIGS[name], seed=3, store_dtype="bfloat16")
        cfg, w = plain.read_model_folder(folder)
        reqs = [replay.random_ids(cfg["vocab_size"], n, 9 + n) for n in (40, 7, 64)]
        ref = [plain.logits(cfg, w, r) for r in reqs]
        rt = GpuRuntime.load(folder, dtype=dtype, max_tokens=64 * 8)
        for r, want in zip(reqs, ref):
            assert rel_err(replay.run_whole(rt, r), want) < VS_PLAIN[dtype]
            assert rel_err(replay.run_tail(rt, r, 8), want) < VS_PLAIN[dtype]
        got, _ = replay.run_batches(rt, reqs, 3, [20, 7, 3])
        for i, want in enumerate(ref):
            assert rel_err(got[i], want) < VS_PLAIN[dtype]
        assert K.bounds_failures() == (0, 0), name
    # a page that was never assigned (-1 in the table): recorded, and nothing is stored for it
    dev = "cuda:0"
    nq, nkv, hd, T = 1, 1, 16, 3
    qkv = torch.randn(T, 3 * hd, device=dev)
    kc = torch.zeros(2, nkv, 64, hd, device=dev); vc = torch.zeros_like(kc)
    table = torch.tensor([[-1, 0]], dtype=torch.int32, device=dev)
    K.rope_cache_write(qkv, torch.arange(T, dtype=torch.int32, device=dev), torch.zeros(0, device=dev), nq, nkv, hd, 0,
                       "half", seq_of_token=torch.zeros(T, dtype=torch.int32, device=dev),
                       slots=torch.zeros(1, dtype=torch.int32, device=dev),
                       len_after=torch.tensor([T], dtype=torch.int32, device=dev), kcache=kc, vcache=vc,
                       page_table=table, ring_rows=0)
    n, index = K.bounds_failures()
    assert n == 1 and index == -1, (n, index)
    assert float(kc.abs().sum()) == 0 and float(vc.abs().sum()) == 0
    assert K.bounds_failures() == (0, 0)               # the record is cleared by reading it
    print("checked build ok")
''')


def test_checked_build_finds_no_bad_index_in_the_engine_and_records_a_planted_one(tmp_path):
    script = SCRIPT.format(root=str(ROOT), tests=str(ROOT / "tests"))
    proc = subprocess.run([sys.executable, "-c", script], capture_output=True, text=True, timeout=1500)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    assert "checked build ok" in proc.stdout


def test_normal_build_has_no_record():
    from airframe_b200 import kernels as K
    assert K.bounds_failures() is None
