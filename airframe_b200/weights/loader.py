"""Weights by tensor name.

Parts declare the tensors they need (:class:`WeightDecl`); the loader checks
the declared set against what a source holds and raises ONE
:class:`WeightError` that lists every missing tensor, every unexpected one and
every wrong shape.  Floating tensors stored in 16 bits are kept in bfloat16, a
tensor stored in 32 bits stays in 32 bits, integer tables become int32; with
``dtype="float32"`` every floating tensor is widened to 32 bits.

Reference: ``MissingTensor`` / ``ShapeMismatch`` of ``src/core/error.rs:26-56``,
the required set of ``src/core/weight_id.rs:112-132`` and its validation in
``src/core/model.rs:1513-1530``.
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


@dataclass
class WeightDecl:
    """A tensor that a part needs.  ``kind`` tells the random-weights mode how
    to fill it: ``matrix`` and ``table`` N(0, 0.02), ``norm`` N(0, 0.1),
    ``int_table`` integers."""
    name: str
    shape: tuple
    kind: str = "matrix"
    optional: bool = False


class WeightError(ValueError):
    """The tensors of a model folder do not match what the model declares."""

    def __init__(self, where, missing=(), unexpected=(), wrong_shape=(), other=()):
        self.missing = list(missing)
        self.unexpected = list(unexpected)
        self.wrong_shape = list(wrong_shape)   # (name, expected, got)
        self.other = list(other)
        lines = [f"{where}: the weights do not match the model"]
        if self.missing:
            lines.append(f"  missing ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        if self.wrong_shape:
            lines.append(f"  wrong shape ({len(self.wrong_shape)}): " + ", ".join(
                f"{n} expected {list(e)} got {list(g)}" for n, e, g in self.wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


class SafetensorsFolder:
    """``model.safetensors``, or the shards named by
    ``model.safetensors.index.json``, of one model folder."""

    def __init__(self, folder):
        self.folder = Path(folder)
        index = self.folder / "model.safetensors.index.json"
        single = self.folder / "model.safetensors"
        self._files = {}
        self._where = {}
        if single.is_file():
            shard_names = [single.name]
        elif index.is_file():
            weight_map = json.loads(index.read_text()).get("weight_map", {})
            shard_names = sorted(set(weight_map.values()))
        else:
            raise WeightError(str(self.folder), other=["no model.safetensors and no model.safetensors.index.json"])
        for shard in shard_names:
            try:
                f = SafetensorsFile(self.folder / shard)
            except (OSError, SafetensorsError) as e:
                raise WeightError(str(self.folder), other=[str(e)]) from e
            self._files[shard] = f
            for n in f.names():
                self._where[n] = f

    def describe(self) -> str:
        return str(self.folder)

    def names(self):
        return list(self._where)

    def info(self, name):
        return self._where[name].info(name)

    def read(self, name, device=None) -> torch.Tensor:
        return self._where[name].read(name)

    def close(self):
        for f in self._files.values():
            f.close()


def kept_dtype(stored: torch.dtype, compute_dtype: torch.dtype) -> torch.dtype:
    """The dtype a stored tensor is kept in."""
    if not stored.is_floating_point:
        return torch.int32
    if compute_dtype == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


def load_weights(source, decls, compute_dtype: torch.dtype, device) -> dict:
    """name -> tensor on ``device`` for every declared tensor that the source holds."""
    if compute_dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"compute dtype must be bfloat16 or float32, got {compute_dtype}")
    have = set(source.names())
    declared = {}
    for d in decls:
        if d.name in declared and tuple(declared[d.name].shape) != tuple(d.shape):
            raise ValueError(f"tensor '{d.name}' is declared twice with different shapes")
        declared.setdefault(d.name, d)
    missing = [n for n, d in declared.items() if n not in have and not d.optional]
    unexpected = sorted(have - set(declared))
    wrong = []
    for n, d in declared.items():
        if n in have:
            _, shape = source.info(n)
            if tuple(shape) != tuple(d.shape):
                wrong.append((n, tuple(d.shape), tuple(shape)))
    if missing or unexpected or wrong:
        raise WeightError(source.describe(), missing, unexpected, wrong)
    out = {}
    for n in declared:
        if n not in have:
            continue
        stored, _ = source.info(n)
        t = source.read(n, device=device)
        out[n] = t.to(device=device, dtype=kept_dtype(stored, compute_dtype)).contiguous()
    return out
