"""Tiny Gemma-2 configurations for the tests.  A and B differ in every size
and option; C has sizes the bfloat16 tensor-core kernels take."""
from __future__ import annotations

import tempfile
from pathlib import Path

TINY_A = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 128, "vocab_size": 256, "rope_theta": 10000.0,
    "sliding_window": 8, "query_pre_attn_scalar": 16, "attn_logit_softcapping": 50.0,
    "final_logit_softcapping": 30.0, "max_position_embeddings": 64, "rms_norm_eps": 1e-6,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "eos_token_id": 1,
    "bos_token_id": 2, "pad_token_id": 0, "torch_dtype": "float32",
}

TINY_B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 320, "vocab_size": 384, "rope_theta": 100000.0,
    "sliding_window": 16, "query_pre_attn_scalar": 24, "attn_logit_softcapping": 20.0,
    "final_logit_softcapping": 15.0, "max_position_embeddings": 128, "rms_norm_eps": 1e-5,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "eos_token_id": [3, 7],
    "bos_token_id": 2, "pad_token_id": 0, "torch_dtype": "float32",
}

# sizes no power of two, head size 48, window that is no multiple of the page
TINY_C = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 4, "hidden_size": 192, "num_attention_heads": 6, "num_key_value_heads": 3,
    "head_dim": 48, "intermediate_size": 448, "vocab_size": 1000, "rope_theta": 5000.0,
    "sliding_window": 40, "query_pre_attn_scalar": 64, "attn_logit_softcapping": 30.0,
    "final_logit_softcapping": 25.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "eos_token_id": 1,
    "torch_dtype": "bfloat16",
}

# the layer widths of Gemma-2 2B (head size 256, 8 heads in 4 groups) with two layers, a small
# vocabulary and a small window: the sizes the tensor-core kernels are tuned for
WIDE_D = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 2304, "num_attention_heads": 8, "num_key_value_heads": 4,
    "head_dim": 256, "intermediate_size": 9216, "vocab_size": 2048, "rope_theta": 10000.0,
    "sliding_window": 100, "query_pre_attn_scalar": 256, "attn_logit_softcapping": 50.0,
    "final_logit_softcapping": 30.0, "max_position_embeddings": 512, "rms_norm_eps": 1e-6,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "eos_token_id": 1,
    "torch_dtype": "bfloat16",
}

# the layer widths of Gemma-2 9B (16 heads in 8 groups, head size 256) and of Gemma-2 27B (32 heads
# in 16 groups, head size 128, a score scale that is not head_dim^-0.5), two layers each
WIDE_E = dict(WIDE_D, hidden_size=3584, num_attention_heads=16, num_key_value_heads=8, intermediate_size=14336,
              vocab_size=1536, sliding_window=72)
WIDE_F = dict(WIDE_D, hidden_size=4608, num_attention_heads=32, num_key_value_heads=16, head_dim=128,
              intermediate_size=36864, query_pre_attn_scalar=144, vocab_size=1024, sliding_window=90)

# sizes that no tensor-core kernel takes: a width that is no multiple of 8, head size 80, five heads
# without grouping, an odd vocabulary, an odd window, no softcaps
ODD_G = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 3, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 80, "intermediate_size": 260, "vocab_size": 777, "rope_theta": 777.0,
    "sliding_window": 33, "query_pre_attn_scalar": 50, "attn_logit_softcapping": None,
    "final_logit_softcapping": None, "max_position_embeddings": 256, "rms_norm_eps": 1e-5,
    "hidden_activation": "gelu_pytorch_tanh", "tie_word_embeddings": True, "eos_token_id": 1,
    "torch_dtype": "bfloat16",
}

# small sizes with head size 128: three query heads on one kv head, a window whose ring wraps
SMALL_H = dict(WIDE_D, num_hidden_layers=3, hidden_size=192, num_attention_heads=3, num_key_value_heads=1,
              head_dim=128, intermediate_size=320, vocab_size=500, sliding_window=70, query_pre_attn_scalar=100,
              attn_logit_softcapping=20.0, rms_norm_eps=1e-5, rope_theta=5000.0)

CONFIGS = {"H": SMALL_H, "A": TINY_A, "B": TINY_B, "C": TINY_C, "D": WIDE_D, "E": WIDE_E, "F": WIDE_F, "G": ODD_G}


def make_folder(cfg_dict, seed=0, store_dtype=None, root=None, device="cpu"):
    """Write a random model folder for ``cfg_dict`` under a temporary place; returns its path."""
    from airframe_b200.config import config_from_dict
    from airframe_b200.weights import write_random_model
    root = Path(root or tempfile.mkdtemp(prefix="af_model_"))
    cfg = config_from_dict(cfg_dict)
    write_random_model(root, cfg, seed, store_dtype or cfg_dict.get("torch_dtype", "bfloat16"), device=device)
    return root
