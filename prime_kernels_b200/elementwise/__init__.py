"""Forward-only CUDA replacements (bf16, sm_100a) for the reference's Triton elementwise ops.

Same call surfaces as ``triton_rope.apply_rotary`` (prime_kernels/triton_rope/__init__.py:373-377),
``triton_rmsnorm.rmsnorm`` / ``residual_rmsnorm`` (prime_kernels/triton_rmsnorm/rmsnorm.py:701-722) and
``triton_swiglu.swiglu`` (prime_kernels/triton_swiglu/swiglu.py:195-202), with the same bf16 rounding points
(those of HuggingFace eager).  Inference path only: no autograd (the backward passes are out of scope),
bf16 only, contiguous inputs.
"""
from __future__ import annotations

import torch

from .._cabi import load_ops

load_ops()

__all__ = ["apply_rotary", "rmsnorm", "residual_rmsnorm", "swiglu"]


@torch.library.register_fake("prime_elementwise::apply_rotary")
def _apply_rotary_fake(q, k, cos, sin, unsqueeze_dim):
    return torch.empty_like(q), torch.empty_like(k)


@torch.library.register_fake("prime_elementwise::rmsnorm")
def _rmsnorm_fake(x, weight, eps):
    return torch.empty_like(x)


@torch.library.register_fake("prime_elementwise::residual_rmsnorm")
def _residual_rmsnorm_fake(branch, residual, weight, eps):
    return torch.empty_like(branch), torch.empty_like(branch)


@torch.library.register_fake("prime_elementwise::swiglu")
def _swiglu_fake(gate, up):
    return torch.empty_like(gate)


def apply_rotary(q, k, cos, sin, unsqueeze_dim: int = 1):
    """Rotate the first ``cos.shape[-1]`` dims of q and k (``[B, heads, S, D]`` for ``unsqueeze_dim=1``,
    ``[B, S, heads, D]`` for 2); cos/sin ``[1 or B, S, rot]``."""
    return torch.ops.prime_elementwise.apply_rotary(q, k, cos, sin, unsqueeze_dim)


def rmsnorm(x, weight, eps: float):
    """RMSNorm over the last dim: ``weight * bf16(x * rstd)``."""
    return torch.ops.prime_elementwise.rmsnorm(x, weight, float(eps))


def residual_rmsnorm(branch, residual, weight, eps: float):
    """``sum = bf16(branch + residual)``; returns ``(rmsnorm(sum), sum)``."""
    return torch.ops.prime_elementwise.residual_rmsnorm(branch, residual, weight, float(eps))


def swiglu(gate, up):
    """``bf16(bf16(silu(gate)) * up)``."""
    return torch.ops.prime_elementwise.swiglu(gate, up)
