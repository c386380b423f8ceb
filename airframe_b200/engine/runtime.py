"""The programming entry point, in the reference's manner:
``GpuRuntime.load(path)`` then ``generate(prompt, SamplingParams)``
(``src/runtime/gpu.rs:94,644-654``; accessors ``:657-733``).  Prompts are token
ids: the library starts where the tokenizer ends.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config import ModelConfig, config_from_folder
from ..weights import RandomSource, SafetensorsFolder, load_weights
from .engine import Engine
from .model import Model

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}

DEFAULT_SAFE_CTX = 8192   # the reference caps the context here unless told otherwise (src/runtime/gpu.rs:203)


def _dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    if name not in _DTYPES:
        raise ValueError(f"dtype must be one of {sorted(_DTYPES)}, got {name!r}")
    return _DTYPES[name]


def _require_gpu(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("airframe_b200 runs on a CUDA device only (no CPU path exists); "
                           f"asked for '{device}', CUDA available: {torch.cuda.is_available()}")
    return device


class GpuRuntime:
    """A loaded model with its cache and generation loop on one GPU."""

    def __init__(self, config: ModelConfig, model: Model, engine: Engine):
        self.config = config
        self.model = model
        self.engine = engine
        self._loop = None

    # ------------------------------------------------------------------ construction

    @classmethod
    def _build(cls, config, source, dtype, device, max_tokens, max_context, max_sequences, spec_edit=None):
        device = _require_gpu(device)
        dt = _dtype(dtype)
        torch.cuda.set_device(device)
        spec = config.model_spec()
        if spec_edit is not None:
            spec_edit(spec)
        model = Model(spec, dt, device)
        model.load(load_weights(source, model.weight_decls(), dt, device))
        limit = model.spec.max_positions
        ctx = min(max_context or DEFAULT_SAFE_CTX, limit)
        engine = Engine(model, max_tokens=max_tokens or ctx, max_context=ctx, max_sequences=max_sequences)
        return cls(config, model, engine)

    @classmethod
    def load(cls, path, dtype="bfloat16", device="cuda:0", max_tokens: Optional[int] = None,
             max_context: Optional[int] = None, max_sequences: Optional[int] = None, spec_edit=None) -> "GpuRuntime":
        """Load a model folder (config.json, model.safetensors).  ``max_tokens``
        sizes the cache: the most tokens that live sequences hold together.
        ``spec_edit(spec)`` may change the :class:`~airframe_b200.config.ModelSpec`
        before the model is built (options of parts that config.json does not carry)."""
        config = config_from_folder(path)
        source = SafetensorsFolder(path)
        try:
            return cls._build(config, source, dtype, device, max_tokens, max_context, max_sequences, spec_edit)
        finally:
            source.close()

    @classmethod
    def random(cls, config: ModelConfig, seed: int = 0, dtype="bfloat16", device="cuda:0",
               max_tokens: Optional[int] = None, max_context: Optional[int] = None,
               max_sequences: Optional[int] = None, on_device: bool = False, spec_edit=None) -> "GpuRuntime":
        """A model of ``config`` with seeded random weights, without a folder.
        ``on_device`` draws them on the GPU (fast for large models; the values
        then differ from a folder written with the same seed)."""
        decls = Model(config.model_spec(), torch.bfloat16, "cpu").weight_decls()
        store = torch.float32 if _dtype(dtype) == torch.float32 else torch.bfloat16
        source = RandomSource(decls, seed, store_dtype=store, device=device if on_device else "cpu")
        return cls._build(config, source, dtype, device, max_tokens, max_context, max_sequences, spec_edit)

    # ------------------------------------------------------------------ use

    def generate(self, prompt, params=None, on_token=None, logits_processor=None):
        """``prompt``: token ids of one request, or a list of such lists.
        Returns the new token ids (a list, or a list of lists).
        ``on_token(request index, token id)`` sees every emitted token;
        ``logits_processor`` is the control hook of
        :mod:`airframe_b200.engine.generate` (the reference's third argument of
        ``generate``, ``src/runtime/gpu.rs:644-654``)."""
        from .generate import GenerationLoop
        from ..sampling import SamplingParams, Sampler
        if self._loop is None:
            self._loop = GenerationLoop(self.engine, Sampler(self.model.spec.vocab_size, self.engine.device),
                                        stop_token_ids=self.model.spec.stop_token_ids)
        params = params or SamplingParams()
        single = len(prompt) > 0 and isinstance(prompt[0], int)
        out = self._loop.generate([list(prompt)] if single else [list(p) for p in prompt], params, on_token,
                                  logits_processor)
        return out[0] if single else out

    def step(self, entries, probe=None):
        return self.engine.step(entries, probe=probe)

    def spec(self):
        return self.model.spec

    def eos_token(self):
        ids = self.model.spec.stop_token_ids
        return ids[0] if ids else None

    def reset(self) -> None:
        """Give back every slot that is still held."""
        for slot in range(self.engine.cache.n_slots):
            if self.engine.cache.slots.is_held(slot):
                self.engine.free_slot(slot)
