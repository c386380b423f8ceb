"""The layers of a decode step as one kernel: the list of phases that
``csrc/decode_layers.cu`` walks, put together from the layers' parts.

A step of few tokens is bound by the weights and cache pages it streams; as
a chain of kernels it also pays every short kernel's fill, drain and memory
round trips.  A :class:`LayerProgram` is the same work as a list of phases
(matrix-vector products with their epilogues, attention over the cache, the
merge of its splits, residual sums with norms) for one persistent kernel whose
copies run ahead across the phases.

The program knows no model: a block that can express itself in phases
implements ``emit_decode`` (see :class:`~airframe_b200.parts.base.Block`) with
the builder methods below; a part that cannot raises
:class:`~airframe_b200.parts.base.NotFusable` and the step runs kernel by
kernel as before.

Reference: the per-layer dispatch of the decode step,
``src/backend/bindless/pipeline/inference.rs:1061-1337`` (one command per
operation there; one kernel for the whole stack here).
"""
from __future__ import annotations

import struct

import numpy as np
import torch

from .. import kernels
from ..kernels_const import PAGE
from ..parts.base import NotFusable

GEMV, ATTN, MERGE, NORM = 0, 1, 2, 3
EP_PARTS, EP_ROPE, EP_GATED = 0, 1, 2
SOURCES = {"normed": 0, "attn_out": 1, "gated": 2}
MAX_K_PARTS = 16


def plan_k_parts(n_tiles: int, k: int, n_blocks: int, kp_max: int, fixed_one: bool = False) -> int:
    """Into how many parts K is cut so that the units (row tile x K part) keep
    all blocks busy: block c works on part c % P and on every (n_blocks // P)-th
    row tile.  The cost of a choice is the columns the busiest block streams,
    plus a little for every partial sum that the next phase has to add."""
    best = None
    for parts in range(1, min(MAX_K_PARTS, n_blocks) + 1):
        if k % parts:
            continue
        kp = k // parts
        if kp % 64 or kp > kp_max:
            continue
        per = n_blocks // parts
        cost = -(-n_tiles // per) * kp + 32 * parts
        if best is None or cost < best[0]:
            best = (cost, parts)
        if fixed_one:
            break
    if best is None or (fixed_one and best[1] != 1):
        raise NotFusable(f"no split of K = {k} into parts of at most {kp_max} columns (multiples of 64)")
    return best[1]


def _ptr_words(t) -> tuple:
    p = 0 if t is None else t.data_ptr()
    return p & 0xFFFFFFFF, p >> 32


def _f32_word(v: float) -> int:
    return struct.unpack("<I", struct.pack("<f", float(v)))[0]


class LayerProgram:
    """Builder, then holder, of one decode step's phases for ``n_tok`` tokens."""

    def __init__(self, n_tok: int, hidden: int, device, max_len_after: int):
        lim = kernels.decode_layers_limits()
        if n_tok > lim["tokens"]:
            raise NotFusable(f"{n_tok} tokens in the step (the kernel takes {lim['tokens']})")
        if hidden > lim["k_part"] or hidden % 64:
            raise NotFusable(f"width {hidden} (a multiple of 64 up to {lim['k_part']})")
        self.lim = lim
        self.n_tok = n_tok
        self.hidden = hidden
        self.device = torch.device(device)
        self.max_len_after = max_len_after
        self.n_blocks = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.words = lim["words"]
        self.phases: list = []
        self.attn: list = []
        self.maps: list = []          # 128-byte tensor maps
        self.keep: list = []          # tensors the program points into
        self.head_dim = None
        self.max_parts = 1
        self.max_inter = 8
        self.max_qwidth = 8
        self.max_split_rows = 1       # (token, head, split) triples of the attention's partial results
        self.rot = 0
        self.finished = False

    # ------------------------------------------------------------------ builder

    def _phase(self, kind: int) -> list:
        w = [0] * self.words
        w[0] = kind
        w[13] = self.rot % self.n_blocks
        self.phases.append(w)
        return w

    def _used(self, n: int) -> None:
        """The next phase's units start at the blocks that this phase left idle."""
        self.rot = (self.rot - min(n, self.n_blocks)) % self.n_blocks

    def _map(self, t, rows: int, cols: int, box_rows: int) -> int:
        self.maps.append(kernels.tensor_map_bf16(t, rows, cols, box_rows))
        self.keep.append(t)
        return len(self.maps) - 1

    def gemv(self, weight, source: str, epilogue: str, attn: int = -1, heads: int = 0, out_rows: int = 0,
             activation: str = "gelu_tanh") -> int:
        """y = W a for the step's tokens.  ``source``: ``normed`` (the last
        norm's output), ``attn_out`` or ``gated``.  ``epilogue``: ``parts``
        (32-bit partial sums per K part, for :meth:`norm`; returns their
        number), ``rope`` (W's rows are ``heads`` heads [q | k | v] of attention
        entry ``attn``: rotation, q to its buffer, k and v to the cache) or
        ``gated`` (W in the gated layout of ``kernels.interleave_gate_up``:
        act(gate) * up into the ``gated`` buffer, ``out_rows`` features)."""
        if weight.dtype != torch.bfloat16 or weight.dim() != 2 or not weight.is_contiguous():
            raise NotFusable("a product's weight must be a contiguous bfloat16 matrix")
        rows, k = weight.shape
        if k % 64 or weight.data_ptr() % 16:
            raise NotFusable(f"a product's K = {k} must be a multiple of 64")
        ep = {"parts": EP_PARTS, "rope": EP_ROPE, "gated": EP_GATED}[epilogue]
        src = SOURCES[source]
        if source == "normed" and k != self.hidden:
            raise NotFusable(f"a product of the normed stream has K = {k}, the width is {self.hidden}")
        if ep == EP_ROPE:
            hd = self.head_dim
            if rows != heads * hd:
                raise NotFusable("the packed q, k, v rows do not match the heads")
            n_tiles = heads * (hd // 32)
        elif ep == EP_GATED:
            if rows % 32 or out_rows > rows // 2:
                raise NotFusable("the gated weight is not in groups of 32 rows")
            n_tiles = rows // 32
            self.max_inter = max(self.max_inter, out_rows)
        else:
            if rows != self.hidden:
                raise NotFusable(f"a product that feeds the residual has {rows} rows, the width is {self.hidden}")
            out_rows = rows
            n_tiles = -(-rows // 32)
        parts = plan_k_parts(n_tiles, k, self.n_blocks, self.lim["k_part"], fixed_one=ep != EP_PARTS)
        w = self._phase(GEMV)
        w[2] = self._map(weight, rows, k, 16)
        w[3], w[4], w[5], w[6] = n_tiles, parts, k // parts, ep
        w[7] = 1 if ep == EP_ROPE else 0
        w[8], w[9], w[10] = src, k, out_rows
        w[11] = kernels.ACTIVATIONS[activation]
        w[12] = max(attn, 0)
        self.max_parts = max(self.max_parts, parts)
        self._used(min(self.n_blocks // parts, n_tiles) * parts)
        return len(self.phases) - 1 if ep == EP_ROPE else parts

    def attention_entry(self, nq: int, nkv: int, hd: int, window: int, kv, scale: float, cap: float, inv_freq) -> int:
        """Registers one layer's attention over its cache view ``kv``; returns its index."""
        if hd not in (128, 256) or (self.head_dim not in (None, hd)):
            raise NotFusable(f"head_dim {hd} (128 or 256, the same in all layers)")
        self.head_dim = hd
        group = nq // nkv
        room = self.lim["attn_bytes"] - 16 * (hd + 8) * 2
        if group > 16 or group * hd * 32 > room:
            raise NotFusable(f"{group} query heads per kv head at head_dim {hd}")
        if kv is None or kv.k is None or kv.k.dtype != torch.bfloat16:
            raise NotFusable("attention without a bfloat16 cache of its own")
        if inv_freq is None or inv_freq.numel() != hd // 2 or inv_freq.dtype != torch.float32:
            raise NotFusable("rotary frequencies for half the head are needed")
        n_pages = kv.k.shape[0]
        if n_pages * nkv * PAGE >= 1 << 31:
            raise NotFusable("the cache has too many rows for one tensor map")
        splits = kernels.attn_decode_splits(self.n_tok, nkv, self.max_len_after, window, blocks=self.n_blocks)
        w = [0] * self.words
        w[0], w[1], w[2], w[3], w[4], w[5] = nq, nkv, window, kv.ring_rows, kv.page_table.shape[1], splits
        w[6], w[7] = _f32_word(scale), _f32_word(cap)
        w[8], w[9] = _ptr_words(kv.k)
        w[10], w[11] = _ptr_words(kv.v)
        w[12], w[13] = _ptr_words(kv.page_table)
        w[14], w[15] = _ptr_words(inv_freq)
        w[16] = self._map(kv.k, n_pages * nkv * PAGE, hd, PAGE)
        self._map(kv.v, n_pages * nkv * PAGE, hd, PAGE)
        self.keep += [kv.page_table, inv_freq]
        self.attn.append(w)
        self.max_qwidth = max(self.max_qwidth, nq * hd)
        self.max_split_rows = max(self.max_split_rows, self.n_tok * nq * splits)
        return len(self.attn) - 1

    def attention(self, attn: int, written_by: int) -> None:
        """Attention of entry ``attn`` over the cache; phase ``written_by`` wrote the new token's row."""
        w = self._phase(ATTN)
        w[12], w[15] = attn, written_by
        e = self.attn[attn]
        self._used(self.n_tok * e[1] * e[5])

    def merge(self, attn: int) -> None:
        w = self._phase(MERGE)
        w[12] = attn
        self._used(self.n_tok * self.attn[attn][0])

    def norm(self, n_parts: int, post, nxt) -> None:
        """x += post(sum of the last product's ``n_parts`` partial sums) (skipped
        when ``n_parts`` is 0), then ``normed`` = nxt(x) (skipped when None)."""
        pp = post.fused_params() if post is not None else None
        pn = nxt.fused_params() if nxt is not None else None
        if (n_parts > 0) != (pp is not None):
            raise NotFusable("a residual sum needs its norm")
        offset = (pp or pn or (None, 0.0, 0.0))[2]
        for p in (pp, pn):
            if p is not None and (p[0].numel() != self.hidden or p[2] != offset or p[0].dtype != torch.float32):
                raise NotFusable("norms of one phase share a weight offset and the stream's width")
        w = self._phase(NORM)
        w[14] = n_parts
        if pp is not None:
            w[16], w[17] = _ptr_words(pp[0])
            w[20] = _f32_word(pp[1])
            self.keep.append(pp[0])
        if pn is not None:
            w[18], w[19] = _ptr_words(pn[0])
            w[21] = _f32_word(pn[1])
            self.keep.append(pn[0])
        w[22] = _f32_word(offset)
        self._used(self.n_tok)

    # ------------------------------------------------------------------ holder

    def finish(self) -> "LayerProgram":
        """Lays the program out on the device."""
        if not self.phases or self.head_dim is None:
            raise NotFusable("an empty program")
        dev = self.device

        def words(rows):
            a = np.array(rows, dtype=np.uint64).astype(np.uint32).view(np.int32)
            return torch.from_numpy(a.copy()).to(dev)

        self.d_phases = words(self.phases)
        self.d_attn = words(self.attn)
        raw = np.frombuffer(b"".join(self.maps), dtype=np.uint8).copy()
        self.d_maps = torch.from_numpy(raw).to(dev)
        if self.d_maps.data_ptr() % 64:
            raise NotFusable("tensor maps are not 64-byte aligned on the device")
        T, H = self.n_tok, self.hidden
        bf = torch.bfloat16
        self.normed = torch.zeros(T, H, dtype=bf, device=dev)
        self.attn_out = torch.zeros(T * self.max_qwidth, dtype=bf, device=dev)
        self.q = torch.zeros(T * self.max_qwidth, dtype=bf, device=dev)
        self.gated = torch.zeros(T * self.max_inter, dtype=bf, device=dev)
        self.parts = torch.zeros(self.max_parts * T * H, dtype=torch.float32, device=dev)
        self.part_o = torch.zeros(self.max_split_rows * self.head_dim, dtype=torch.float32, device=dev)
        self.part_ml = torch.zeros(self.max_split_rows * 2, dtype=torch.float32, device=dev)
        self.sync = torch.zeros(2, dtype=torch.int32, device=dev)
        self.finished = True
        return self

    def run(self, x, batch) -> None:
        """Runs the phases on the residual stream x (float32 [n_tok, hidden], in place)."""
        if not self.finished:
            raise RuntimeError("the program is not finished")
        if tuple(x.shape) != (self.n_tok, self.hidden) or x.dtype != torch.float32 or not x.is_contiguous():
            raise kernels.KernelError("LayerProgram.run: x must be a contiguous float32 [tokens, width]")
        kernels.decode_layers(self, x, batch.positions, batch.slots, batch.len_after)

    @property
    def n_phases(self) -> int:
        return len(self.phases)

    def describe(self) -> str:
        names = {GEMV: "product", ATTN: "attention", MERGE: "merge", NORM: "norm"}
        out = []
        for i, w in enumerate(self.phases):
            s = f"{i}: {names[w[0]]}"
            if w[0] == GEMV:
                s += f" tiles {w[3]} x K parts {w[4]} of {w[5]} columns, epilogue {w[6]}"
            out.append(s)
        return "\n".join(out)

