"""The model's two ends: the token embedding and the head that makes logits.

Embedding: row gather times ``scale`` (reference: row fetch
``src/runtime/gpu.rs:420-431``, sqrt(hidden) factor
``src/bin/shimmy_server_gpu/server_inference.rs:603-609``).  Head: row dots
with the head matrix, then the final softcap, logits in float32 (reference:
``src/backend/bindless/sh_head_blob.wgsl:300-334``; tied to the embedding when
no separate matrix exists, ``src/runtime/gpu.rs:763-795``).
"""
from __future__ import annotations

import torch

from .. import kernels
from ..weights.loader import WeightDecl
from .base import Part, register_part
from .linear import linear


@register_part("embedding", "token_embedding")
class TokenEmbedding(Part):
    """Parameters: ``weight``, ``vocab_size``, ``hidden_size``, ``scale``."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.name = self.param("weight")
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.scale = float(self.param("scale"))
        self.table = None

    def weight_decls(self):
        return [WeightDecl(self.name, (self.vocab, self.hidden), "table")]

    def load(self, weights):
        self.table = weights[self.name].to(self.ctx.compute_dtype).contiguous()

    def decode_bytes(self, lens) -> int:
        return len(lens) * self.hidden * (4 if self.ctx.compute_dtype == torch.float32 else 2)   # the rows it gathers

    def forward(self, ids):
        """ids int32 [T] -> float32 residual stream [T, H]."""
        x = torch.empty(ids.shape[0], self.hidden, dtype=torch.float32, device=ids.device)
        kernels.embed(x, self.table, ids, self.scale)
        return x


@register_part("head", "lm_head")
class LmHead(Part):
    """Parameters: ``vocab_size``, ``hidden_size``, ``softcap`` (0 = off) and
    either ``weight`` or ``tied_to`` (+ ``optional_weight`` that wins when the
    folder holds it)."""
    graph_safe = True


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.vocab = int(self.param("vocab_size"))
        self.hidden = int(self.param("hidden_size"))
        self.softcap = float(self.params.get("softcap") or 0.0)
        self.w = None
        self._keys = None      # the fused arg-max's key per row (zero between calls)

    def weight_decls(self):
        shape = (self.vocab, self.hidden)
        if "weight" in self.params:
            return [WeightDecl(self.params["weight"], shape, "table")]
        decls = [WeightDecl(self.param("tied_to"), shape, "table")]
        if self.params.get("optional_weight"):
            decls.append(WeightDecl(self.params["optional_weight"], shape, "table", optional=True))
        return decls

    def load(self, weights):
        name = self.params.get("weight") or self.params.get("optional_weight")
        if name is None or name not in weights:
            name = self.param("tied_to")
        self.w = weights[name].to(self.ctx.compute_dtype).contiguous()

    def decode_bytes(self, lens) -> int:
        return self.vocab * self.hidden * (4 if self.ctx.compute_dtype == torch.float32 else 2)

    def logits_flops(self, rows: int) -> int:
        return 2 * rows * self.vocab * self.hidden

    def forward(self, y):
        """y [R, H] compute dtype (after the final norm) -> float32 logits [R, V]."""
        return linear(y, self.w, out_dtype=torch.float32, cap=self.softcap)

    def forward_argmax(self, y):
        """The token of greedy decoding for every row: int32 [R], the arg-max of
        the (capped) logits over finite values, the lowest id among equals.
        On the tensor-core path the logits never go to memory (the product's
        epilogue keeps the best per row); else logits and the sampler's arg-max."""
        R = y.shape[0]
        tokens = torch.empty(R, dtype=torch.int32, device=y.device)
        if kernels.gemm_tc_supported(y, self.w, None):
            stride = kernels.argmax_key_stride()
            if self._keys is None or self._keys.numel() < R * stride:
                self._keys = torch.zeros(max(R, 256) * stride, dtype=torch.int64, device=y.device)
            kernels.gemm_tc_argmax(tokens, y, self.w, self.softcap, self._keys)
        else:
            kernels.sample(self.forward(y), tokens, 0.0, 1.0, 1.0)
        return tokens
