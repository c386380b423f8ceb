"""Named configurations for the random-weights mode: the two tiny test
models and the layer sizes of the released Gemma-2 models, as config.json
dictionaries.  Nothing here is read by the model code: a configuration always
reaches it through ``config_from_dict``."""
from __future__ import annotations

_COMMON = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2", "hidden_activation": "gelu_pytorch_tanh",
    "tie_word_embeddings": True, "rms_norm_eps": 1e-6,
}

PRESETS = {
    "tinyA": dict(_COMMON, num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                  head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0, sliding_window=8,
                  query_pre_attn_scalar=16, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                  max_position_embeddings=64, torch_dtype="float32"),
    "tinyB": dict(_COMMON, num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=1,
                  head_dim=32, intermediate_size=320, vocab_size=384, rope_theta=100000.0, sliding_window=16,
                  query_pre_attn_scalar=24, attn_logit_softcapping=20.0, final_logit_softcapping=15.0,
                  max_position_embeddings=128, torch_dtype="float32"),
    "2b": dict(_COMMON, num_hidden_layers=26, hidden_size=2304, num_attention_heads=8, num_key_value_heads=4,
               head_dim=256, intermediate_size=9216, vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
               query_pre_attn_scalar=256, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
               max_position_embeddings=8192, torch_dtype="bfloat16"),
    "9b": dict(_COMMON, num_hidden_layers=42, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8,
               head_dim=256, intermediate_size=14336, vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
               query_pre_attn_scalar=256, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
               max_position_embeddings=8192, torch_dtype="bfloat16"),
    "27b": dict(_COMMON, num_hidden_layers=46, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16,
                head_dim=128, intermediate_size=36864, vocab_size=256000, rope_theta=10000.0, sliding_window=4096,
                query_pre_attn_scalar=144, attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                max_position_embeddings=8192, torch_dtype="bfloat16"),
}


def preset(name: str) -> dict:
    """The config.json dictionary of a named configuration (a copy)."""
    if name not in PRESETS:
        raise KeyError(f"unknown preset '{name}' (known: {', '.join(sorted(PRESETS))})")
    return dict(PRESETS[name])
