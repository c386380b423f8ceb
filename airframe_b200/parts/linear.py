"""y = x W^T for a weight [out, in]: picks the matrix-product kernel.

float32: the plain CUDA-core kernel (true 32-bit).  bfloat16: the tensor-core
kernels where they take the sizes, the plain kernel (bfloat16 operands, 32-bit
accumulators) otherwise.
"""
from __future__ import annotations

import torch

from .. import kernels


def linear(x, w, out_dtype=None, cap: float = 0.0, out=None):
    """x [M, K] (dense rows), w [N, K] -> [M, N] in ``out_dtype`` (x's by default).
    ``cap`` > 0 applies the softcap cap * tanh(y / cap) to the result."""
    M = x.shape[0]
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or x.dtype, device=x.device)
    if kernels.gemm_tc_supported(x, w, out):
        kernels.gemm_tc(out, x, w, cap, checked=True)
    else:
        kernels.gemm_plain(out, x, w, cap)
    return out


class PartialSums:
    """The result of a product as float32 split-K partial sums [S, M, N]; the
    consumer (a norm's ``add_normed``, the rotary kernel) adds them in order."""

    def __init__(self, parts):
        self.parts = parts

    @property
    def shape(self):
        return self.parts.shape[1:]


def linear_split(x, w):
    """x w^T for few rows and a long K: split-K partial sums when that fills
    the GPU better, else the plain result.  Returns a tensor or PartialSums."""
    M, K = x.shape
    N = w.shape[0]
    if kernels.gemm_tc_supported(x, w, None):
        splits = kernels.gemm_tc_splits(M, N, K)
        if splits > 1:
            parts = torch.empty(splits, M, N, dtype=torch.float32, device=x.device)
            kernels.gemm_tc(parts, x, w, splits=splits, checked=True)
            return PartialSums(parts)
        out = torch.empty(M, N, dtype=x.dtype, device=x.device)
        kernels.gemm_tc(out, x, w, checked=True)
        return out
    return linear(x, w)


def gated_linear(x, w_gu, inter: int, activation: str, interleaved: bool):
    """act(x w_gate^T) * (x w_up^T).  ``interleaved``: w_gu is in the gated
    tensor-core layout (``kernels.interleave_gate_up``) and one kernel with the
    activation in its epilogue does it all; else w_gu = [gate rows; up rows],
    a product and the activation kernel."""
    M = x.shape[0]
    out = torch.empty(M, inter, dtype=x.dtype, device=x.device)
    if interleaved:
        full = out if w_gu.shape[0] // 2 == inter else torch.empty(M, w_gu.shape[0] // 2, dtype=x.dtype, device=x.device)
        kernels.gemm_tc(full, x, w_gu, gated=True, activation=activation)
        return full if full is out else full[:, :inter].contiguous()
    gu = linear(x, w_gu)
    kernels.gated_act(out, gu, activation)
    return out
