"""The safetensors container, loading by name and its one error, random weights (no GPU)."""
import json
import struct

import pytest
import torch

from airframe_b200.config import config_from_dict
from airframe_b200.engine import declared_weights
from airframe_b200.weights import (RandomSource, SafetensorsError, SafetensorsFile, SafetensorsFolder,
                                   WeightDecl, WeightError, kept_dtype, load_weights, write_random_model,
                                   write_safetensors)
from tiny import TINY_A, TINY_B, make_folder
import plain_gemma2 as plain


def _write(path, tensors):
    write_safetensors(path, [(n, tuple(t.shape), t.dtype, (lambda t=t: t)) for n, t in tensors.items()])


def test_container_round_trip(tmp_path):
    ts = {"a": torch.randn(3, 5).to(torch.bfloat16), "b": torch.arange(7, dtype=torch.int64),
          "c": torch.randn(2, 2, 2), "e": torch.empty(0, 4)}
    _write(tmp_path / "x.safetensors", ts)
    f = SafetensorsFile(tmp_path / "x.safetensors")
    assert sorted(f.names()) == sorted(ts)
    for n, t in ts.items():
        assert f.info(n) == (t.dtype, tuple(t.shape))
        assert torch.equal(f.read(n), t)
    # the plain implementation's own reader sees the same bytes
    mine = plain.read_safetensors(tmp_path / "x.safetensors")
    assert all(torch.equal(mine[n], t) for n, t in ts.items())
    f.close()


def test_container_errors(tmp_path):
    p = tmp_path / "bad.safetensors"
    p.write_bytes(b"abc")
    with pytest.raises(SafetensorsError, match="too short"):
        SafetensorsFile(p)
    p.write_bytes(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(SafetensorsError, match="header length"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 8)          # data cut short
    with pytest.raises(SafetensorsError, match="outside the file"):
        SafetensorsFile(p)
    hdr = json.dumps({"w": {"dtype": "F8_E4M3", "shape": [4], "data_offsets": [0, 4]}}).encode()
    p.write_bytes(struct.pack("<Q", len(hdr)) + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="unsupported dtype"):
        SafetensorsFile(p)


def test_declared_tensors_of_tiny_a():
    decls = declared_weights(config_from_dict(TINY_A).model_spec())
    names = {d.name: d for d in decls}
    assert names["model.embed_tokens.weight"].shape == (256, 64)
    assert names["model.layers.1.self_attn.k_proj.weight"].shape == (32, 64)
    assert names["model.layers.0.mlp.down_proj.weight"].shape == (64, 128)
    assert names["model.layers.0.pre_feedforward_layernorm.weight"].kind == "norm"
    assert names["lm_head.weight"].optional and not names["model.embed_tokens.weight"].optional
    assert len([d for d in decls if not d.optional]) == 2 + 2 * 11


def test_random_folder_is_seeded_and_loadable(tmp_path):
    a = make_folder(TINY_A, seed=3, root=tmp_path / "a")
    b = make_folder(TINY_A, seed=3, root=tmp_path / "b")
    c = make_folder(TINY_A, seed=4, root=tmp_path / "c")
    wa, wb, wc = (plain.read_safetensors(x / "model.safetensors") for x in (a, b, c))
    assert all(torch.equal(wa[k], wb[k]) for k in wa)
    assert not torch.equal(wa["model.norm.weight"], wc["model.norm.weight"])
    m = wa["model.layers.0.mlp.up_proj.weight"].float()
    n = torch.cat([wa[k].float() for k in wa if k.endswith("layernorm.weight")])
    assert 0.015 < m.std() < 0.025 and 0.07 < n.std() < 0.13
    decls = declared_weights(config_from_dict(TINY_A).model_spec())
    src = SafetensorsFolder(a)
    w = load_weights(src, decls, torch.bfloat16, "cpu")
    assert "lm_head.weight" not in w and len(w) == len(wa)
    assert json.loads((a / "config.json").read_text())["architectures"] == ["Gemma2ForCausalLM"]
    # the same tensors without a folder
    rs = RandomSource(decls, 3, store_dtype=torch.float32)
    assert torch.equal(rs.read("model.norm.weight"), wa["model.norm.weight"])


def test_dtype_policy(tmp_path):
    assert kept_dtype(torch.bfloat16, torch.bfloat16) == torch.bfloat16
    assert kept_dtype(torch.float16, torch.bfloat16) == torch.bfloat16
    assert kept_dtype(torch.float32, torch.bfloat16) == torch.float32      # stored in 32 bits: stays so
    assert kept_dtype(torch.bfloat16, torch.float32) == torch.float32
    assert kept_dtype(torch.int64, torch.bfloat16) == torch.int32
    ts = {"m": torch.randn(4, 4).to(torch.bfloat16), "n": torch.randn(4), "t": torch.arange(4)}
    _write(tmp_path / "model.safetensors", ts)
    decls = [WeightDecl("m", (4, 4)), WeightDecl("n", (4,), "norm"), WeightDecl("t", (4,), "int_table")]
    w = load_weights(SafetensorsFolder(tmp_path), decls, torch.bfloat16, "cpu")
    assert (w["m"].dtype, w["n"].dtype, w["t"].dtype) == (torch.bfloat16, torch.float32, torch.int32)
    w = load_weights(SafetensorsFolder(tmp_path), decls, torch.float32, "cpu")
    assert (w["m"].dtype, w["n"].dtype, w["t"].dtype) == (torch.float32, torch.float32, torch.int32)


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(TINY_B, seed=1, root=tmp_path)
    w = plain.read_safetensors(folder / "model.safetensors")
    del w["model.layers.1.mlp.up_proj.weight"]
    del w["model.norm.weight"]
    w["model.layers.9.extra.weight"] = torch.zeros(2)
    w["model.layers.0.self_attn.q_proj.weight"] = torch.zeros(10, 96)
    _write(folder / "model.safetensors", w)
    decls = declared_weights(config_from_dict(TINY_B).model_spec())
    with pytest.raises(WeightError) as ei:
        load_weights(SafetensorsFolder(folder), decls, torch.bfloat16, "cpu")
    e = ei.value
    assert sorted(e.missing) == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert e.wrong_shape == [("model.layers.0.self_attn.q_proj.weight", (192, 96), (10, 96))]
    text = str(e)
    for word in ("missing (2)", "unexpected (1)", "wrong shape (1)", "expected [192, 96] got [10, 96]",
                 "model.norm.weight", "model.layers.9.extra.weight"):
        assert word in text


def test_folder_without_weights(tmp_path):
    with pytest.raises(WeightError, match="no model.safetensors"):
        SafetensorsFolder(tmp_path)
    (tmp_path / "model.safetensors").write_bytes(b"12")
    with pytest.raises(WeightError, match="too short"):
        SafetensorsFolder(tmp_path)


def test_sharded_folder(tmp_path):
    _write(tmp_path / "s1.safetensors", {"a": torch.ones(2)})
    _write(tmp_path / "s2.safetensors", {"b": torch.zeros(3)})
    (tmp_path / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "s1.safetensors", "b": "s2.safetensors"}}))
    w = load_weights(SafetensorsFolder(tmp_path), [WeightDecl("a", (2,)), WeightDecl("b", (3,))],
                     torch.float32, "cpu")
    assert w["a"].sum() == 2 and w["b"].shape == (3,)
