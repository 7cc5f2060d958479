"""CUDA replacements (bf16, sm_100a) for the reference's Triton elementwise ops, forward and backward.

Same call surfaces as ``triton_rope.apply_rotary`` (prime_kernels/triton_rope/__init__.py:373-377),
``triton_rmsnorm.rmsnorm`` / ``residual_rmsnorm`` (prime_kernels/triton_rmsnorm/rmsnorm.py:701-722) and
``triton_swiglu.swiglu`` (prime_kernels/triton_swiglu/swiglu.py:195-202), with the same bf16 rounding points
(those of HuggingFace eager / PyTorch autograd on the fp32-upcast reference).  Autograd goes through q, k
(rotary), x / branch / residual and weight (norms), gate and up (SwiGLU), like the reference's autograd functions
(triton_rope/__init__.py:353-370, triton_rmsnorm/rmsnorm.py:502-698, triton_swiglu/swiglu.py:149-192); cos / sin
and eps get no gradient.  bf16 only, contiguous inputs (SwiGLU rows may be strided).
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


@torch.library.register_fake("prime_elementwise::apply_rotary_backward")
def _apply_rotary_backward_fake(grad_q, grad_k, cos, sin, unsqueeze_dim):
    return torch.empty_like(grad_q), torch.empty_like(grad_k)


@torch.library.register_fake("prime_elementwise::rmsnorm_backward")
def _rmsnorm_backward_fake(grad_out, grad_sum, x, weight, eps):
    return torch.empty_like(x), torch.empty_like(weight)


@torch.library.register_fake("prime_elementwise::swiglu_backward")
def _swiglu_backward_fake(grad, gate, up):
    return torch.empty_like(gate), torch.empty_like(gate)


# ---- autograd: the backward of each op is another op of this library
def _rotary_setup(ctx, inputs, output):
    _, _, cos, sin, unsqueeze_dim = inputs
    ctx.save_for_backward(cos, sin)
    ctx.unsqueeze_dim = unsqueeze_dim


def _rotary_backward(ctx, grad_q, grad_k):
    cos, sin = ctx.saved_tensors
    if grad_q is None and grad_k is None:
        return None, None, None, None, None
    dq, dk = torch.ops.prime_elementwise.apply_rotary_backward(grad_q.contiguous(), grad_k.contiguous(), cos, sin,
                                                               ctx.unsqueeze_dim)
    return dq, dk, None, None, None


def _rmsnorm_setup(ctx, inputs, output):
    x, weight, eps = inputs
    ctx.save_for_backward(x, weight)
    ctx.eps = eps


def _rmsnorm_backward(ctx, grad_out):
    x, weight = ctx.saved_tensors
    dx, dw = torch.ops.prime_elementwise.rmsnorm_backward(grad_out.contiguous(), None, x, weight, ctx.eps)
    return dx, dw, None


def _residual_rmsnorm_setup(ctx, inputs, output):
    _, _, weight, eps = inputs
    ctx.save_for_backward(output[1], weight)          # the sum is the normed input
    ctx.eps = eps
    ctx.set_materialize_grads(False)


def _residual_rmsnorm_backward(ctx, grad_out, grad_sum):
    summed, weight = ctx.saved_tensors
    if grad_out is None:
        if grad_sum is None:
            return None, None, None, None
        return grad_sum, grad_sum, None, None       # only the sum was used downstream
    dx, dw = torch.ops.prime_elementwise.rmsnorm_backward(grad_out.contiguous(),
                                                          None if grad_sum is None else grad_sum.contiguous(), summed,
                                                          weight, ctx.eps)
    return dx, dx, dw, None


def _swiglu_setup(ctx, inputs, output):
    ctx.save_for_backward(*inputs)


def _swiglu_backward(ctx, grad):
    gate, up = ctx.saved_tensors
    return torch.ops.prime_elementwise.swiglu_backward(grad, gate, up)


torch.library.register_autograd("prime_elementwise::apply_rotary", _rotary_backward, setup_context=_rotary_setup)
torch.library.register_autograd("prime_elementwise::rmsnorm", _rmsnorm_backward, setup_context=_rmsnorm_setup)
torch.library.register_autograd("prime_elementwise::residual_rmsnorm", _residual_rmsnorm_backward,
                                setup_context=_residual_rmsnorm_setup)
torch.library.register_autograd("prime_elementwise::swiglu", _swiglu_backward, setup_context=_swiglu_setup)


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
