"""A per-layer localizer: facts of the residual stream after every scheduled
run of a step, small enough to print and to compare with another
implementation's, so that a run that drifts names the layer where it starts.

Per run and wanted row: the root mean square, the first values and a checksum
(the 32-bit patterns of the row's floats added as 64-bit integers).
Reference: ``LayerTrace`` / ``TokenTrace`` (``src/debug_trace.rs:75-125``), the
per-stage RMS of ``src/bin/invariant_probe.rs:1-20`` and the checksum of
``crates/airframe_observe/src/facts.rs:361-374``.

A probed step runs kernel by kernel (never as a captured graph) and copies the
rows it looks at to the host after every run: a tool for finding faults, not a
path of generation.
"""
from __future__ import annotations

import numpy as np
import torch


def row_facts(row, first: int = 20) -> dict:
    """RMS, first values and bit-sum checksum of one float32 row (a numpy array)."""
    row = np.ascontiguousarray(row, dtype=np.float32)
    bits = row.view(np.uint32).astype(np.int64)
    return {"rms": float(np.sqrt(np.mean(row.astype(np.float64) ** 2))) if row.size else 0.0,
            "first": [float(v) for v in row[:first]],
            "checksum": int(bits.sum())}


class LayerProbe:
    """Pass one to ``Engine.step(..., probe=...)``.  ``rows``: the rows of the
    step (indices into its tokens, sequence after sequence) to look at; by
    default the rows whose logits are wanted, or all rows when none is."""

    def __init__(self, rows=None, first: int = 20):
        self.rows = None if rows is None else [int(r) for r in rows]
        self.first = int(first)
        self.records: list = []

    def _rows_of(self, batch):
        if self.rows is not None:
            return torch.tensor(self.rows, dtype=torch.long, device=batch.tokens.device)
        if batch.want_rows is not None:
            return batch.want_rows.long()
        return torch.arange(batch.n_tokens, device=batch.tokens.device)

    def after(self, run: int, layer: int, x, batch) -> None:
        """``x``: the float32 residual stream [T, H] once run ``run`` (of layer
        ``layer``; -1: the embedding) is done."""
        data = x.index_select(0, self._rows_of(batch)).to(torch.float32).cpu().numpy()
        self.records.append({"run": run, "layer": layer, "rows": [row_facts(r, self.first) for r in data]})

    def to_json(self) -> list:
        return self.records


def first_difference(records, reference, tolerance: float):
    """The first run whose facts differ from another implementation's by more
    than ``tolerance`` (relative), as (run, layer, row), or None.
    ``reference[run][row]`` is that implementation's float row (any sequence of
    floats, at least as long as the recorded first values): the RMS of the
    whole row is compared and, value by value, its first elements (relative to
    the largest of them)."""
    for rec in records:
        if rec["run"] < 0 or rec["run"] >= len(reference):
            continue
        for r, facts in enumerate(rec["rows"]):
            ref = np.asarray(reference[rec["run"]][r], dtype=np.float64)
            ref_rms = float(np.sqrt(np.mean(ref ** 2)))
            if abs(facts["rms"] - ref_rms) > tolerance * max(ref_rms, 1e-30):
                return rec["run"], rec["layer"], r
            got = np.asarray(facts["first"], dtype=np.float64)
            want = ref[: got.size]
            if got.size and float(np.abs(got - want).max()) > tolerance * max(float(np.abs(want).max()), 1e-30):
                return rec["run"], rec["layer"], r
    return None
