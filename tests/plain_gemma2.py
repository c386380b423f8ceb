"""Plain, slow Gemma-2 written from the reference's formulas.

Whole sequences, dense masks, no cache, float64 by default, one function for
each part.  It shares no code with ``airframe_b200``: it has its own
config reading, its own safetensors reader and its own sampling.  Nothing
here was compared with the reference's compiled code: the reference is a Rust
crate whose CPU model is Llama-only and whose GPU path needs a graphics API,
so this file rests on the formulas in the reference's sources, cited by
``file:line`` (paths inside the reference project) at each function.

Where the reference deviates from Gemma-2 as its weights in Hugging Face
layout expect it (no ``query_pre_attn_scalar``, no alternating window, GGUF
norm weights that already hold ``1 + w``, adjacent-pair RoPE for permuted
GGUF q/k rows), the Gemma-2 behaviour is used and the docstring says so.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

# --------------------------------------------------------------------------
# model folder reading (own code; the product's loader is not used)
# --------------------------------------------------------------------------

_ST_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16,
    "BF16": torch.bfloat16, "I64": torch.int64, "I32": torch.int32,
}


def read_safetensors(path, dtype=None) -> dict:
    """name -> torch tensor (CPU) of one .safetensors file, in the stored dtype or
    widened to ``dtype`` (each tensor is converted straight from the file's bytes)."""
    raw = np.fromfile(str(path), dtype=np.uint8)
    (hlen,) = struct.unpack("<Q", raw[:8].tobytes())
    header = json.loads(raw[8:8 + hlen].tobytes().decode("utf-8"))
    base = 8 + hlen
    whole = torch.from_numpy(raw)
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        a, b = meta["data_offsets"]
        dt = _ST_DTYPES[meta["dtype"]]
        chunk = whole[base + a: base + b]
        if (base + a) % torch.empty(0, dtype=dt).element_size():
            chunk = chunk.clone()                              # (a view of wider elements must start aligned)
        t = chunk.view(dt) if b > a else torch.empty(0, dtype=dt)
        t = t.reshape(meta["shape"])
        out[name] = t.to(dtype) if dtype is not None and t.is_floating_point() else t.clone()
    return out


def read_model_folder(folder, dtype=torch.float64):
    """(config dict, weights dict widened to ``dtype``)."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = read_safetensors(folder / "model.safetensors", dtype)
    return cfg, w


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------

def embed(ids, table, hidden_size):
    """Row gather, then times sqrt(hidden).

    Reference: row fetch ``src/runtime/gpu.rs:420-431``; the sqrt(H) factor is
    applied in ``src/bin/shimmy_server_gpu/server_inference.rs:603-609``
    (``emb_scale = sqrt(n_embd)``); the hook is ``embedding_scale()`` in
    ``src/family/mod.rs:56-59``.  Applied always here.
    """
    ids = torch.as_tensor(ids, dtype=torch.long)
    return table[ids] * math.sqrt(float(hidden_size))


def rms_norm(x, w, eps):
    """y = x * rsqrt(mean(x^2) + eps) * (1 + w).

    Reference: ``src/backend/bindless/sh_layer_v1.wgsl:426-451`` (sum of
    squares over the row / dim, inverseSqrt(ms + eps), times weight) and
    ``src/backend/bindless/sh_rmsnorm.wgsl:69-93``.  The reference multiplies
    by the stored weight because GGUF files hold ``1 + w`` already
    (``src/backend/bindless/preflight.rs:199-205`` copies it verbatim);
    weights under Hugging Face names hold ``w``, so the factor is ``1 + w``.
    """
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * (1.0 + w)


def rope_angles(positions, head_dim, theta):
    """angle[t, p] = pos_t * theta^(-2p/head_dim), p < head_dim/2.

    Reference: ``src/backend/bindless/preflight.rs:87-90`` (theta_p =
    base^(-2p/rope_dim)), table by distance ``:102-111``.
    """
    p = torch.arange(head_dim // 2, dtype=torch.float64)
    inv_freq = torch.as_tensor(float(theta), dtype=torch.float64) ** (-2.0 * p / head_dim)
    pos = torch.as_tensor(positions, dtype=torch.float64)
    return pos[:, None] * inv_freq[None, :]


def rope(x, positions, theta):
    """Rotate x[T, heads, head_dim] by absolute position, pairs (i, i + hd/2).

    Reference: the score-time relative rotation of
    ``src/backend/bindless/sh_layer_v1.wgsl:706-725`` equals rotating q by its
    position and k by its own; the absolute form is
    ``src/ops/reference/rope.rs:156-196``.  The reference pairs adjacent
    elements (2p, 2p+1) because GGUF q/k rows are permuted; weights in
    Hugging Face layout pair element i with i + head_dim/2, used here.
    """
    T, n, hd = x.shape
    ang = rope_angles(positions, hd, theta).to(x.dtype)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    x1, x2 = x[..., : hd // 2], x[..., hd // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


def softcap(s, cap):
    """cap * tanh(s / cap) when cap > 0.

    Reference: ``src/backend/bindless/sh_layer_v1.wgsl:727-730`` (scores),
    ``src/backend/bindless/sh_head_blob.wgsl:329-332`` (logits).
    """
    if cap is None or cap <= 0:
        return s
    return cap * torch.tanh(s / cap)


def visibility(T, window):
    """mask[i, j] = key j visible to query i.

    Causal: ``src/backend/bindless/sh_layer_v1.wgsl:693`` (skip pos > own
    position).  The reference has no per-layer window; Gemma-2's local layers
    see key j iff j <= i and i - j < sliding_window.
    """
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if window is not None:
        m = m & ((i - j) < window)
    return m


def attention(q, k, v, scale, cap, window):
    """q[T, nq, hd], k/v[T, nkv, hd] (already rotated) -> ctx[T, nq*hd].

    Reference: ``src/backend/bindless/sh_layer_v1.wgsl:662-754``: score =
    dot * scale (``:726``), softcap (``:727-730``), softmax over visible keys
    (online form ``:739-745``, normalised ``:749-753``), times V; query head h
    reads kv head h / (nq/nkv) (``:673,677``).  The reference fixes scale at
    head_dim^-0.5 (``:674``); Gemma-2 uses query_pre_attn_scalar^-0.5.
    """
    T, nq, hd = q.shape
    nkv = k.shape[1]
    group = nq // nkv
    mask = visibility(T, window)
    out = torch.empty(T, nq, hd, dtype=q.dtype)
    for h in range(nq):
        g = h // group
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = softcap(s, cap)
        s = s.masked_fill(~mask, float("-inf"))
        p = torch.softmax(s, dim=-1)
        out[:, h, :] = p @ v[:, g, :]
    return out.reshape(T, nq * hd)


def gelu_tanh(g):
    """0.5 g (1 + tanh(0.7978845608 (g + 0.044715 g^3))).

    Reference: ``src/backend/bindless/sh_layer_v1.wgsl:1079``.
    """
    return 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g * g * g)))


def geglu_mlp(n2, w_gate, w_up, w_down):
    """f = W_down (gelu_tanh(W_gate n2) * (W_up n2)); weights are [out, in].

    Reference: ``src/backend/bindless/sh_layer_v1.wgsl:1024-1070`` (gate, up
    row dots), ``:1079`` (activation), ``:1104-1140`` (down).
    """
    return (gelu_tanh(n2 @ w_gate.T) * (n2 @ w_up.T)) @ w_down.T


def is_sliding(layer):
    """Gemma-2 alternation: even layers are local (layer 0 sliding, 1 global)."""
    return layer % 2 == 0


def block(x, positions, layer, cfg, w):
    """One decoder layer on x[T, H] of one sequence.

    Reference order ``src/backend/bindless/pipeline/inference.rs:1096-1251``:
    attn_norm, q/k/v, attention, o-proj, post-attention norm and residual
    (net x + norm(a), ``sh_layer_v1.wgsl:811-813,834-849``), ffn norm, gate/up
    with activation, down, post-ffw norm and residual (``:869-884,1147-1148``).
    """
    pre = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    nq, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    T = x.shape[0]
    n1 = rms_norm(x, w[pre + "input_layernorm.weight"], eps)
    q = (n1 @ w[pre + "self_attn.q_proj.weight"].T).reshape(T, nq, hd)
    k = (n1 @ w[pre + "self_attn.k_proj.weight"].T).reshape(T, nkv, hd)
    v = (n1 @ w[pre + "self_attn.v_proj.weight"].T).reshape(T, nkv, hd)
    q = rope(q, positions, cfg["rope_theta"])
    k = rope(k, positions, cfg["rope_theta"])
    window = cfg["sliding_window"] if is_sliding(layer) else None
    ctx = attention(q, k, v, float(cfg["query_pre_attn_scalar"]) ** -0.5,
                    cfg.get("attn_logit_softcapping"), window)
    a = ctx @ w[pre + "self_attn.o_proj.weight"].T
    x = x + rms_norm(a, w[pre + "post_attention_layernorm.weight"], eps)
    n2 = rms_norm(x, w[pre + "pre_feedforward_layernorm.weight"], eps)
    f = geglu_mlp(n2, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"],
                  w[pre + "mlp.down_proj.weight"])
    return x + rms_norm(f, w[pre + "post_feedforward_layernorm.weight"], eps)


def hidden_states(cfg, w, ids, upto_layer=None):
    """Residual stream after ``upto_layer`` layers (all by default), [T, H]."""
    x = embed(ids, w["model.embed_tokens.weight"], cfg["hidden_size"])
    positions = list(range(len(ids)))
    n = cfg["num_hidden_layers"] if upto_layer is None else upto_layer
    for layer in range(n):
        x = block(x, positions, layer, cfg, w)
    return x


def lm_head(x, cfg, w):
    """Final norm, tied head, final softcap -> logits[T, V].

    Reference: final norm ``src/backend/bindless/sh_rmsnorm.wgsl:69-93``; head
    row dots and cap ``src/backend/bindless/sh_head_blob.wgsl:300-334``; the
    head is the embedding when no separate output tensor exists
    (``src/runtime/gpu.rs:763-795``).
    """
    y = rms_norm(x, w["model.norm.weight"], cfg["rms_norm_eps"])
    head = w.get("lm_head.weight", w["model.embed_tokens.weight"])
    return softcap(y @ head.T, cfg.get("final_logit_softcapping"))


def logits(cfg, w, ids):
    """Logits at every position of one whole sequence, [T, V]."""
    return lm_head(hidden_states(cfg, w, ids), cfg, w)


# --------------------------------------------------------------------------
# sampling (reference: src/runtime/gpu.rs)
# --------------------------------------------------------------------------

_MASK64 = (1 << 64) - 1


class XorShift64Star:
    """``src/runtime/gpu.rs:50-62``: state = seed + 1; u = (x * M >> 40) / 2^24."""

    def __init__(self, seed):
        self.s = (seed + 1) & _MASK64

    def next_f32(self):
        s = self.s
        s ^= s >> 12
        s ^= (s << 25) & _MASK64
        s ^= s >> 27
        self.s = s
        val = (s * 0x2545F4914F6CDD1D) & _MASK64
        return np.float32(val >> 40) / np.float32(16777216.0)


def greedy(row):
    """Arg-max over finite logits, lowest index on ties.

    Reference: CPU sampler ``src/runtime/sampling.rs:50-58`` (first max wins).
    """
    row = np.asarray(row, dtype=np.float32)
    best, idx = -np.inf, 0
    for i, v in enumerate(row):
        if np.isfinite(v) and v > best:
            best, idx = v, i
    return idx


def apply_repetition_penalty(row, recent, penalty):
    """``src/runtime/gpu.rs:889-900``: logit > 0 ? / p : * p, once per listed token."""
    row = np.array(row, dtype=np.float32)
    if penalty != 1.0:
        for tok in recent:
            if 0 <= tok < row.shape[0]:
                row[tok] = row[tok] / np.float32(penalty) if row[tok] > 0 else row[tok] * np.float32(penalty)
    return row


def sample_token(row, temperature, top_p, repetition_penalty, recent, u):
    """``src/runtime/gpu.rs:880-962`` with the uniform draw ``u`` given.

    Penalty, then greedy when temperature < 1e-7, else logits / T, softmax,
    sort descending, smallest prefix whose sum reaches top_p, r = u * prefix
    sum, first index whose running sum reaches r.
    """
    row = apply_repetition_penalty(row, recent, repetition_penalty)
    if temperature < 1e-7:
        return greedy(row)
    z = np.where(np.isfinite(row), row * np.float32(1.0 / temperature), -np.inf).astype(np.float32)
    p = np.exp(z - z.max()).astype(np.float32)
    p = p / p.sum(dtype=np.float32)
    order = np.argsort(-p, kind="stable")
    cum = np.float32(0.0)
    cutoff = len(order)
    for i, idx in enumerate(order):
        cum = np.float32(cum + p[idx])
        if cum >= np.float32(top_p):
            cutoff = i + 1
            break
    nucleus = order[:cutoff]
    nsum = np.float32(0.0)
    for idx in nucleus:
        nsum = np.float32(nsum + p[idx])
    r = np.float32(u) * nsum
    acc = np.float32(0.0)
    for idx in nucleus:
        acc = np.float32(acc + p[idx])
        if acc >= r:
            return int(idx)
    return int(nucleus[-1])


def generate_greedy(cfg, w, prompt, max_tokens, stop_ids=()):
    """Greedy chain by whole-sequence recomputation; stop token not emitted
    (``crates/airframe_observe/src/isf.rs:397-410,477-485``)."""
    ids = list(prompt)
    out = []
    for _ in range(max_tokens):
        row = logits(cfg, w, ids)[-1].to(torch.float32).numpy()
        t = greedy(row)
        if t in stop_ids:
            break
        out.append(t)
        ids.append(t)
    return out
