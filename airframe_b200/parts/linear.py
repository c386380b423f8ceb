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
    if x.dtype == torch.bfloat16 and kernels.gemm_bf16_supported(M, N, x.shape[1], x, w, out):
        kernels.gemm_bf16(out, x, w, cap)
    else:
        kernels.gemm_plain(out, x, w, cap)
    return out
