"""Fused RMSNorm + residual + MXFP8 quantisation (sm_100a).

Same surface as the reference package (prime_kernels/rmsnorm/__init__.py:33-53 in the reference
project): ``fused_rmsnorm_residual(branch, residual, weight, epsilon=1e-6)`` returning
``(vals, scales, rrms)``, registered as ``torch.ops.prime_rmsnorm.fused_rmsnorm_residual`` with a
fake kernel for tracing.  Shapes are relaxed: N is arbitrary and C only has to be a multiple of 32;
scale bytes of partially covered 128x128 tiles are written as 0.
"""
from __future__ import annotations

import torch

from .._cabi import load_ops

load_ops()

__all__ = ["fused_rmsnorm_residual", "fused_rmsnorm_residual_ex", "SCALE_TILE_BYTES"]

# One 512 byte scale tile per 128 row x 128 column block.
SCALE_TILE_BYTES = 512
_SCALE_TILE = SCALE_TILE_BYTES


def _scale_numel(n: int, c: int) -> int:
    return ((n + 127) // 128) * ((c + 127) // 128) * _SCALE_TILE


@torch.library.register_fake("prime_rmsnorm::fused_rmsnorm_residual")
def _fused_rmsnorm_residual_fake(branch, residual, weight, epsilon):
    n, c = branch.shape
    device = branch.device
    return (
        torch.empty((n, c), dtype=torch.float8_e4m3fn, device=device),
        torch.empty(_scale_numel(n, c), dtype=torch.float8_e8m0fnu, device=device),
        torch.empty(n, dtype=torch.float32, device=device),
    )


@torch.library.register_fake("prime_rmsnorm::fused_rmsnorm_residual_ex")
def _fused_rmsnorm_residual_ex_fake(branch, residual, weight, epsilon, residual_out, prenorm_add):
    n, c = branch.shape
    device = branch.device
    return (
        torch.empty((n, c), dtype=torch.float8_e4m3fn, device=device),
        torch.empty(_scale_numel(n, c), dtype=torch.float8_e8m0fnu, device=device),
        torch.empty(n, dtype=torch.float32, device=device),
        torch.empty((n, c) if residual_out else (0,), dtype=torch.bfloat16, device=device),
    )


def fused_rmsnorm_residual(branch: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                           epsilon: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """RMSNorm over ``branch``, ``residual`` added after the norm, output quantised to MXFP8.

    ``branch`` and ``residual`` are bf16 ``(N, C)``, ``weight`` is bf16 ``(C,)``.  Returns
    ``(vals, scales, rrms)``: ``vals`` fp8 e4m3 ``(N, C)``; ``scales`` flat e8m0, one exponent per 32
    values in the blocked layout a block-scaled tensor-core GEMM reads (512-byte tiles, each covering
    128 rows x 128 columns, ``ceil(N/128) * ceil(C/128)`` of them); ``rrms`` fp32 ``(N,)``.
    """
    return torch.ops.prime_rmsnorm.fused_rmsnorm_residual(branch, residual, weight, epsilon)


def fused_rmsnorm_residual_ex(branch: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor,
                              epsilon: float = 1e-6, *, residual_out: bool = False, prenorm_add: bool = False):
    """Extended op: ``(vals, scales, rrms, updated_residual_or_None)``.

    ``prenorm_add=False``: same maths as :func:`fused_rmsnorm_residual`; the optional fourth output is
    the bf16 value that was quantised.  ``prenorm_add=True``: ``sum = bf16(branch + residual)`` is
    normalised (``bf16(rrms * (sum * weight))``) and quantised; the fourth output is ``sum``.
    """
    vals, scales, rrms, res = torch.ops.prime_rmsnorm.fused_rmsnorm_residual_ex(
        branch, residual, weight, epsilon, residual_out, prenorm_add)
    return vals, scales, rrms, (res if residual_out else None)
