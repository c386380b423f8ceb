"""Seeded random weights: a source that makes each declared tensor from
(seed, tensor name), and a writer of whole model folders (config.json and
model.safetensors).  Matrices and tables are N(0, 0.02), norm weights
N(0, 0.1) (they act as ``offset + w``).

The reference has no such mode (its tests use zeros and ones,
``src/family/llama.rs:625-682``).
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .loader import WeightDecl
from .safetensors_io import write_safetensors

_STD = {"matrix": 0.02, "table": 0.02, "norm": 0.1}
_STORE = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(decl: WeightDecl, seed: int, dtype: torch.dtype, device="cpu") -> torch.Tensor:
    """The tensor of ``decl`` for ``seed``.  Values depend on the device kind
    (the CPU and CUDA generators differ); folders are always written from the CPU."""
    gen = torch.Generator(device=device)
    gen.manual_seed(tensor_seed(seed, decl.name))
    if decl.kind == "int_table":
        return torch.randint(0, 1 << 15, tuple(decl.shape), generator=gen, device=device, dtype=torch.int32)
    if decl.kind not in _STD:
        raise ValueError(f"tensor '{decl.name}': unknown kind '{decl.kind}'")
    t = torch.empty(tuple(decl.shape), dtype=torch.float32, device=device)
    t.normal_(0.0, _STD[decl.kind], generator=gen)
    return t.to(dtype)


class RandomSource:
    """A weight source that holds exactly the declared tensors."""

    def __init__(self, decls, seed: int, store_dtype=torch.bfloat16, device="cpu"):
        self.decls = {d.name: d for d in decls if not d.optional}
        self.seed = seed
        self.store_dtype = store_dtype
        self.device = device

    def describe(self) -> str:
        return f"random weights (seed {self.seed})"

    def names(self):
        return list(self.decls)

    def info(self, name):
        d = self.decls[name]
        return (torch.int32 if d.kind == "int_table" else self.store_dtype), tuple(d.shape)

    def read(self, name, device=None) -> torch.Tensor:
        return random_tensor(self.decls[name], self.seed, self.store_dtype, self.device)


def write_random_model(folder, config, seed: int, store_dtype: str = "bfloat16", device="cpu") -> Path:
    """Write ``config.json`` and ``model.safetensors`` with seeded random
    weights for ``config`` (a typed configuration of a registered architecture).
    ``device``: where the values are drawn (a CUDA device draws billions of
    values in seconds; its values differ from the CPU's for the same seed)."""
    from ..engine.model import declared_weights  # late: the engine imports this package

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    dtype = _STORE[store_dtype]
    data = config.to_dict()
    data["torch_dtype"] = store_dtype
    (folder / "config.json").write_text(json.dumps(data, indent=1))
    decls = [d for d in declared_weights(config.model_spec()) if not d.optional]

    def entries():
        for d in decls:
            dt = torch.int32 if d.kind == "int_table" else dtype
            yield d.name, tuple(d.shape), dt, (lambda d=d: random_tensor(d, seed, dtype, device))

    write_safetensors(folder / "model.safetensors", entries(), metadata={"format": "pt", "seed": seed})
    return folder
