"""Typed reading of ``config.json`` and the generic description of a model.

A configuration class of one architecture reads its own keys with
:class:`KeyReader` (typed, with one error that names the key) and turns
itself into a :class:`ModelSpec`: per-layer part descriptions and the order
in which layers run.  The engine builds models from a ``ModelSpec`` only and
knows no architecture.

Counterpart in the reference: ``ModelSpec`` (``src/core/spec.rs:78-161``) and
the per-layer switches of ``LayerParams``
(``src/backend/bindless/pipeline/mod.rs:77-120``).
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Optional


class ConfigError(ValueError):
    """A key of config.json is missing, of the wrong type or out of range."""


_MISSING = object()


class KeyReader:
    """Typed access to the keys of one config.json dictionary."""

    def __init__(self, data: dict, where: str = "config.json"):
        if not isinstance(data, dict):
            raise ConfigError(f"{where}: expected an object, got {type(data).__name__}")
        self.data = data
        self.where = where

    def _get(self, key: str, default):
        if key not in self.data or self.data[key] is None:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing")
            return default
        return self.data[key]

    def integer(self, key: str, default=_MISSING, minimum: Optional[int] = None) -> int:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, int):
            if isinstance(v, float) and v.is_integer():
                v = int(v)
            else:
                raise ConfigError(f"{self.where}: key '{key}' must be an integer, got {v!r}")
        if minimum is not None and v < minimum:
            raise ConfigError(f"{self.where}: key '{key}' must be >= {minimum}, got {v}")
        return v

    def number(self, key: str, default=_MISSING, positive: bool = False) -> float:
        v = self._get(key, default)
        if v is default and default is not _MISSING:
            return v
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"{self.where}: key '{key}' must be a number, got {v!r}")
        v = float(v)
        if positive and not v > 0:
            raise ConfigError(f"{self.where}: key '{key}' must be > 0, got {v}")
        return v

    def optional_number(self, key: str, default=_MISSING) -> Optional[float]:
        """A number, or ``None`` when the key is null.  An absent key gives
        ``default``; without one the key must be there (null is an answer,
        silence is not)."""
        if key not in self.data:
            if default is _MISSING:
                raise ConfigError(f"{self.where}: required key '{key}' is missing (write null to switch it off)")
            return default
        if self.data[key] is None:
            return None
        return self.number(key)

    def boolean(self, key: str, default=_MISSING) -> bool:
        v = self._get(key, default)
        if not isinstance(v, bool):
            raise ConfigError(f"{self.where}: key '{key}' must be true or false, got {v!r}")
        return v

    def string(self, key: str, default=_MISSING) -> str:
        v = self._get(key, default)
        if not isinstance(v, str):
            raise ConfigError(f"{self.where}: key '{key}' must be a string, got {v!r}")
        return v

    def id_list(self, key: str) -> list[int]:
        """An id or a list of ids; empty when absent or null."""
        v = self.data.get(key)
        if v is None:
            return []
        items = v if isinstance(v, list) else [v]
        for x in items:
            if isinstance(x, bool) or not isinstance(x, int):
                raise ConfigError(f"{self.where}: key '{key}' must hold integer ids, got {v!r}")
        return list(items)


# --------------------------------------------------------------------------
# generic model description
# --------------------------------------------------------------------------

@dataclass
class PartSpec:
    """One part: its kind (a name in the part registry) and its parameters."""
    kind: str
    params: dict = field(default_factory=dict)


@dataclass
class LayerSpec:
    """One layer: where its weights live and which parts it is made of.

    ``norms`` maps a role of the block arrangement (for example ``pre_mixer``)
    to a norm part; the arrangement says which roles it wants.
    """
    prefix: str
    block: PartSpec
    mixer: PartSpec
    feed_forward: PartSpec
    norms: dict


@dataclass
class ScheduleEntry:
    """One run of a layer.  ``cache_from`` names an earlier entry of the
    schedule whose cache this run reads instead of keeping one of its own."""
    layer: int
    cache_from: Optional[int] = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: list
    schedule: list
    final_norm: PartSpec
    head: PartSpec
    stop_token_ids: list = field(default_factory=list)

    def validate(self) -> None:
        if not self.layers:
            raise ConfigError("a model needs at least one layer")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ConfigError(f"schedule entry {i} names layer {e.layer} of {len(self.layers)}")
            if e.cache_from is not None:
                if not 0 <= e.cache_from < i:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_from}, "
                                      "which does not come before it")
                if self.schedule[e.cache_from].cache_from is not None:
                    raise ConfigError(f"schedule entry {i} reads the cache of entry {e.cache_from}, "
                                      "which keeps none itself")


class ModelConfig:
    """Base of the typed configurations.  A subclass sets ``architecture``,
    reads its keys in ``from_dict`` and describes the model in ``model_spec``."""

    architecture: str = ""

    @classmethod
    def from_dict(cls, data: dict) -> "ModelConfig":
        raise NotImplementedError

    def to_dict(self) -> dict:
        raise NotImplementedError

    def model_spec(self) -> ModelSpec:
        raise NotImplementedError


def read_config_json(folder) -> dict:
    path = Path(folder) / "config.json"
    if not path.is_file():
        raise ConfigError(f"{path}: no such file")
    try:
        data = json.loads(path.read_text())
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON: {e}") from e
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: expected an object")
    return data
