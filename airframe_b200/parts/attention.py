"""Grouped-query attention over the paged cache, with score scale, softcap
and an optional window.

score = softcap(q.k * scale), softmax over the visible keys in 32 bits, times
v; query head h reads key/value head h // (heads / kv_heads).  Reference:
``src/backend/bindless/sh_layer_v1.wgsl:662-754`` (scale ``:726``, cap
``:727-730``, online softmax ``:739-753``, head mapping ``:673,677``), the
projections ``:499-530`` and ``:775-804``.  The reference fixes the scale at
head_dim^-0.5 and has no window; both are parameters here.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import ConfigError, PartSpec
from ..weights.loader import WeightDecl
from .base import KVNeed, Mixer, build_part, register_part
from .linear import PartialSums, linear_split


@register_part("mixer", "attention")
class Attention(Mixer):
    """Parameters: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``,
    ``scale``, ``softcap`` (0 = off), ``window`` (None = all keys), ``position``
    (a PartSpec of category ``position``), ``q_weight``/``k_weight``/``v_weight``/
    ``o_weight`` (tensor names); optional ``rope_epilogue`` (default false): run the
    q, k, v projection with the rotary encoding and the cache write in its epilogue
    (``kernels.gemm_tc_rope``) where sizes and encoding allow.  Off by default
    because it measures slower than the projection followed by the rotary kernel:
    four epilogue warps a block cannot hide the latency of the table of cosines
    that many blocks of the rotary kernel hide easily (Gemma-2 2B sizes: a
    2,048-token prompt 9.6 ms against 8.3, a decode step at batch 8 1.93 ms against 1.75)."""

    @property
    def graph_safe(self):
        return self.position.graph_safe


    def __init__(self, params, ctx):
        super().__init__(params, ctx)
        self.hidden = int(self.param("hidden_size"))
        self.nq = int(self.param("num_heads"))
        self.nkv = int(self.param("num_kv_heads"))
        self.hd = int(self.param("head_dim"))
        self.scale = float(self.param("scale"))
        self.softcap = float(self.params.get("softcap") or 0.0)
        w = self.params.get("window")
        self.window = int(w) if w else None
        if self.nq % self.nkv:
            raise ConfigError(f"attention: {self.nq} heads are not a multiple of {self.nkv} kv heads")
        pos = self.params.get("position") or PartSpec("none")
        self.position = build_part("position", pos, ctx)
        self.names = [self.param(k) for k in ("q_weight", "k_weight", "v_weight", "o_weight")]
        self.w_qkv = None
        self.w_o = None
        self.rope_epilogue = False

    def kv_need(self):
        return KVNeed(self.nkv, self.hd, self.window)

    def weight_decls(self):
        q, k, v, o = self.names
        return [WeightDecl(q, (self.nq * self.hd, self.hidden)),
                WeightDecl(k, (self.nkv * self.hd, self.hidden)),
                WeightDecl(v, (self.nkv * self.hd, self.hidden)),
                WeightDecl(o, (self.hidden, self.nq * self.hd)),
                *self.position.weight_decls()]

    def load(self, weights):
        q, k, v, o = self.names
        dt = self.ctx.compute_dtype
        # one matrix product for q, k and v: rows [q heads | k heads | v heads]
        self.w_qkv = torch.cat([weights[q], weights[k], weights[v]], dim=0).to(dt).contiguous()
        self.w_o = weights[o].to(dt).contiguous()
        self.position.load(weights)
        # bfloat16 with a head size and a K that the tensor-core product takes: the rows of every head in the
        # order in which the product's epilogue rotates pairs and writes the cache (used only when the position
        # encoding says, step by step, that it is such a rotation)
        self.rope_epilogue = (bool(self.params.get("rope_epilogue")) and dt == torch.bfloat16 and self.hd % 32 == 0
                              and self.hidden % 8 == 0 and self.w_qkv.is_cuda
                              and self.position.rotates_half_pairs(self.hd))
        if self.rope_epilogue:
            order = kernels.rope_row_order(self.nq + 2 * self.nkv, self.hd, self.w_qkv.device)
            self.w_qkv = self.w_qkv.index_select(0, order).contiguous()
            self.tickets = torch.zeros(4 * ((self.w_qkv.shape[0] + 127) // 128), dtype=torch.int32,
                                       device=self.w_qkv.device)

    def _el(self) -> int:
        return 4 if self.ctx.compute_dtype == torch.float32 else 2

    def decode_bytes(self, lens) -> int:
        weights = ((self.nq + 2 * self.nkv) * self.hd * self.hidden + self.hidden * self.nq * self.hd) * self._el()
        kv_row = 2 * self.nkv * self.hd * self._el()
        return weights + sum(kv_row * (min(n, self.window) if self.window else n) for n in lens)

    def score_flops(self, lens) -> int:
        """The part of :meth:`prefill_flops` that is scores and their products with v."""
        pairs = 0
        for n in lens:          # visible (query, key) pairs of a causal prompt, with the window where there is one
            w = self.window
            pairs += n * (n + 1) // 2 if not w or n <= w else w * (w + 1) // 2 + (n - w) * w
        return 2 * 2 * pairs * self.nq * self.hd

    def prefill_flops(self, lens) -> int:
        T = sum(lens)
        proj = 2 * T * ((self.nq + 2 * self.nkv) * self.hd * self.hidden + self.hidden * self.nq * self.hd)
        return proj + self.score_flops(lens)

    def _project_rotate_store(self, x, batch, view):
        """q, k, v rows of the step with positions encoded and k, v stored: the
        product with the rotation and the cache write in its epilogue."""
        nq, nkv, hd = self.nq, self.nkv, self.hd
        table = self.position.rotary_table(batch, hd)
        M, N = x.shape[0], self.w_qkv.shape[0]
        rows = kc = vc = None
        if view.writes:
            kv = view.kv
            key = ("kv_rows", kv.page_table.data_ptr(), kv.ring_rows, nkv)
            if key not in batch.aux:
                batch.aux[key] = kernels.kv_rows(batch, kv, nkv)
            rows, kc, vc = batch.aux[key], kv.k, kv.v
        qkv = torch.empty(M, N, dtype=x.dtype, device=x.device)
        splits = kernels.gemm_tc_splits(M, N, x.shape[1]) if M <= 64 else 1
        kernels.gemm_tc_rope(qkv, x, self.w_qkv, table, nq, nkv, hd, rows, kc, vc, splits=splits,
                             tickets=self.tickets)
        return qkv

    def forward(self, x, batch, view):
        nq, nkv, hd = self.nq, self.nkv, self.hd
        kv = view.kv
        if self.rope_epilogue:
            qkv = self._project_rotate_store(x, batch, view)
        else:
            qkv = linear_split(x, self.w_qkv)
            parts = None
            if isinstance(qkv, PartialSums):
                parts = qkv.parts
                qkv = torch.empty(x.shape[0], (nq + 2 * nkv) * hd, dtype=x.dtype, device=x.device)
            # positions into q and k, then k and v into the cache: the store is this mixer's; an encoding
            # that can do both in one kernel says so
            if not view.writes:
                self.position.encode(qkv, batch, nq, nkv, hd, parts=parts)
            elif not self.position.encode_and_store(qkv, batch, nq, nkv, hd, kv, parts=parts):
                self.position.encode(qkv, batch, nq, nkv, hd, parts=parts)
                kernels.store_kv(qkv, batch, nq, nkv, hd, kv)
        slopes = self.position.score_slopes(nq)
        q = qkv[:, : nq * hd]
        k = qkv[:, nq * hd: (nq + nkv) * hd]
        v = qkv[:, (nq + nkv) * hd:]
        ctx = torch.empty(x.shape[0], nq * hd, dtype=x.dtype, device=x.device)
        window = self.window or 0
        if batch.is_prefill:
            if not view.writes:
                k, v = batch.step_kv[view.cache_id]
            elif view.keep_step_kv:
                batch.step_kv[view.cache_id] = (k.clone(), v.clone())
            kernels.attn_prefill(ctx, q, k, v, batch, nq, nkv, hd, self.scale, self.softcap, window, slopes)
        else:
            kernels.attn_decode(ctx, q, kv, batch, nq, nkv, hd, self.scale, self.softcap, window, slopes)
        return linear_split(ctx, self.w_o)
