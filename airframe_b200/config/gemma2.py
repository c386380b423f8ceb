"""Gemma-2 (``Gemma2ForCausalLM``): its config.json keys and its layers.

Every size and constant comes from config.json.  What is fixed here is what
config.json does not carry: the alternation of local and global layers (even
layers local) when ``layer_types`` is absent, the half-split rotary pairing of
weights in Hugging Face layout, the ``1 + w`` norm weights and the tensor
names.

Reference: the Gemma-2 switches of the GPU path: post norms
(``src/core/spec.rs:140``), softcaps (``src/core/spec.rs:272-281``), tanh-GELU
gate (``src/backend/bindless/sh_layer_v1.wgsl:1073-1079``), embedding scale
(``src/bin/shimmy_server_gpu/server_inference.rs:603-609``).  The reference
lacks ``query_pre_attn_scalar`` and per-layer windows; both are read here.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Optional

from .base import (ConfigError, KeyReader, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                   ScheduleEntry)

_ACTIVATIONS = {"gelu_pytorch_tanh": "gelu_tanh"}
_LAYER_TYPES = {"sliding_attention": True, "full_attention": False}


@dataclass
class Gemma2Config(ModelConfig):
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    intermediate_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    sliding_window: int
    query_pre_attn_scalar: float
    attn_logit_softcapping: Optional[float]
    final_logit_softcapping: Optional[float]
    hidden_activation: str = "gelu_pytorch_tanh"
    tie_word_embeddings: bool = True
    layer_types: list = field(default_factory=list)   # True = sliding, per layer
    bos_token_id: Optional[int] = None
    eos_token_ids: list = field(default_factory=list)
    pad_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    architecture = "Gemma2ForCausalLM"

    @classmethod
    def from_dict(cls, data: dict) -> "Gemma2Config":
        r = KeyReader(data)
        nq = r.integer("num_attention_heads", minimum=1)
        hd = r.integer("head_dim", minimum=1)
        n_layers = r.integer("num_hidden_layers", minimum=1)
        act = r.string("hidden_activation", r.string("hidden_act", "gelu_pytorch_tanh"))
        if act not in _ACTIVATIONS:
            raise ConfigError(f"config.json: hidden_activation '{act}' is not supported "
                              f"(known: {sorted(_ACTIVATIONS)})")
        if "attention_bias" in data and data["attention_bias"]:
            raise ConfigError("config.json: attention_bias = true is not supported")
        if "layer_types" in data and data["layer_types"] is not None:
            names = data["layer_types"]
            if not isinstance(names, list) or len(names) != n_layers:
                raise ConfigError(f"config.json: layer_types must list {n_layers} layers")
            try:
                layer_types = [_LAYER_TYPES[n] for n in names]
            except (KeyError, TypeError):
                raise ConfigError(f"config.json: layer_types holds an unknown kind "
                                  f"(known: {sorted(_LAYER_TYPES)})") from None
        else:
            layer_types = [layer % 2 == 0 for layer in range(n_layers)]
        bos = r.id_list("bos_token_id")
        pad = r.id_list("pad_token_id")
        cfg = cls(
            vocab_size=r.integer("vocab_size", minimum=1),
            hidden_size=r.integer("hidden_size", minimum=1),
            num_hidden_layers=n_layers,
            intermediate_size=r.integer("intermediate_size", minimum=1),
            num_attention_heads=nq,
            num_key_value_heads=r.integer("num_key_value_heads", nq, minimum=1),
            head_dim=hd,
            rms_norm_eps=r.number("rms_norm_eps", positive=True),
            rope_theta=r.number("rope_theta", positive=True),
            max_position_embeddings=r.integer("max_position_embeddings", minimum=1),
            sliding_window=r.integer("sliding_window", minimum=1),
            query_pre_attn_scalar=r.number("query_pre_attn_scalar", float(hd), positive=True),
            # no value of its own stands here for a cap: the key says a number or null (off); a folder
            # that leaves it out is refused rather than run with another model's logits
            attn_logit_softcapping=r.optional_number("attn_logit_softcapping"),
            final_logit_softcapping=r.optional_number("final_logit_softcapping"),
            hidden_activation=act,
            tie_word_embeddings=r.boolean("tie_word_embeddings", True),
            layer_types=layer_types,
            bos_token_id=bos[0] if bos else None,
            eos_token_ids=r.id_list("eos_token_id"),
            pad_token_id=pad[0] if pad else None,
            torch_dtype=r.string("torch_dtype", r.string("dtype", "bfloat16")),
        )
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(f"config.json: num_attention_heads {self.num_attention_heads} is not a "
                              f"multiple of num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2 != 0:
            raise ConfigError(f"config.json: head_dim {self.head_dim} must be even for rotary pairs")
        for key in ("attn_logit_softcapping", "final_logit_softcapping"):
            v = getattr(self, key)
            if v is not None and v < 0:
                raise ConfigError(f"config.json: {key} must be >= 0 or null, got {v}")
        for t in self.eos_token_ids:
            if not 0 <= t < self.vocab_size:
                raise ConfigError(f"config.json: eos_token_id {t} outside the vocabulary")
        if len(self.layer_types) != self.num_hidden_layers:
            raise ConfigError("layer_types must have one entry per layer")

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "gemma2"
        d["layer_types"] = ["sliding_attention" if s else "full_attention" for s in self.layer_types]
        eos = d.pop("eos_token_ids")
        d["eos_token_id"] = eos[0] if len(eos) == 1 else (eos or None)
        d["hidden_act"] = self.hidden_activation
        # other readers of this layout want an integer here when the value is one
        if float(self.query_pre_attn_scalar).is_integer():
            d["query_pre_attn_scalar"] = int(self.query_pre_attn_scalar)
        return d

    # ----------------------------------------------------------------------

    def model_spec(self) -> ModelSpec:
        h = self.hidden_size

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"weight": name, "size": h, "eps": self.rms_norm_eps,
                                         "weight_offset": 1.0})

        layers = []
        for i in range(self.num_hidden_layers):
            p = f"model.layers.{i}."
            rope = PartSpec("rope", {"theta": self.rope_theta, "rotary_dim": self.head_dim,
                                     "pairing": "half"})
            mixer = PartSpec("attention", {
                "hidden_size": h,
                "num_heads": self.num_attention_heads,
                "num_kv_heads": self.num_key_value_heads,
                "head_dim": self.head_dim,
                "scale": float(self.query_pre_attn_scalar) ** -0.5,
                "softcap": self.attn_logit_softcapping or 0.0,
                "window": self.sliding_window if self.layer_types[i] else None,
                "position": rope,
                "q_weight": p + "self_attn.q_proj.weight",
                "k_weight": p + "self_attn.k_proj.weight",
                "v_weight": p + "self_attn.v_proj.weight",
                "o_weight": p + "self_attn.o_proj.weight",
            })
            ffn = PartSpec("gated_mlp", {
                "hidden_size": h,
                "intermediate_size": self.intermediate_size,
                "activation": _ACTIVATIONS[self.hidden_activation],
                "gate_weight": p + "mlp.gate_proj.weight",
                "up_weight": p + "mlp.up_proj.weight",
                "down_weight": p + "mlp.down_proj.weight",
            })
            norms = {
                "pre_mixer": norm(p + "input_layernorm.weight"),
                "post_mixer": norm(p + "post_attention_layernorm.weight"),
                "pre_feed_forward": norm(p + "pre_feedforward_layernorm.weight"),
                "post_feed_forward": norm(p + "post_feedforward_layernorm.weight"),
            }
            layers.append(LayerSpec(prefix=p, block=PartSpec("sandwich"), mixer=mixer,
                                    feed_forward=ffn, norms=norms))
        head_params = {"vocab_size": self.vocab_size, "hidden_size": h,
                       "softcap": self.final_logit_softcapping or 0.0}
        if self.tie_word_embeddings:
            head_params["tied_to"] = "model.embed_tokens.weight"
            head_params["optional_weight"] = "lm_head.weight"
        else:
            head_params["weight"] = "lm_head.weight"
        spec = ModelSpec(
            architecture=self.architecture,
            hidden_size=h,
            vocab_size=self.vocab_size,
            max_positions=self.max_position_embeddings,
            embedding=PartSpec("token_embedding", {"weight": "model.embed_tokens.weight",
                                                   "vocab_size": self.vocab_size, "hidden_size": h,
                                                   "scale": math.sqrt(float(h))}),
            layers=layers,
            schedule=[ScheduleEntry(i) for i in range(self.num_hidden_layers)],
            final_norm=norm("model.norm.weight"),
            head=PartSpec("lm_head", head_params),
            stop_token_ids=list(self.eos_token_ids),
        )
        spec.validate()
        return spec
