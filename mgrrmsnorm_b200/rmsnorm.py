"""RMSNorm module and autograd Function: the host-side mirror of megagemm/rmsnorm.py.

Same names, constructor arguments, parameter name (`weight`, so state dicts load) and error
behaviour as the reference (megagemm/rmsnorm.py:18-78); the arithmetic is in libmgr_b200.so.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from . import rmsnorm_cuda_ops


class RMSNormFunction(torch.autograd.Function):
    """Autograd Function over rmsnorm_forward / rmsnorm_backward (megagemm/rmsnorm.py:18-48)."""

    @staticmethod
    def forward(ctx, input: torch.Tensor, weight: torch.Tensor, epsilon: float = 1e-5):
        orig_shape = input.shape
        # a view, as in the reference (:28): a non-viewable input raises instead of being copied
        input_2d = input.view(-1, input.size(-1))
        output, inv_rms = rmsnorm_cuda_ops.rmsnorm_forward(input_2d, weight, epsilon)
        ctx.save_for_backward(input_2d, weight, inv_rms)
        ctx.epsilon = epsilon
        ctx.orig_shape = orig_shape
        return output.view(orig_shape)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        input_2d, weight, inv_rms = ctx.saved_tensors
        grad_output_2d = grad_output.contiguous().view(-1, grad_output.size(-1))
        grad_input, grad_weight = rmsnorm_cuda_ops.rmsnorm_backward(grad_output_2d, input_2d, weight, inv_rms)
        return grad_input.view(ctx.orig_shape), grad_weight, None


class RMSNorm(nn.Module):
    """Root-mean-square layer norm, y = x * rsqrt(mean(x^2, -1) + epsilon) * weight.

    Args (as megagemm/rmsnorm.py:68): hidden_size, epsilon (default 1e-5). `weight` starts at ones in
    fp32; call `.half()` / `.to(torch.bfloat16)` on the module to match a half-precision input, as with
    the reference (input and weight share one dtype).
    """

    def __init__(self, hidden_size: int, epsilon: float = 1e-5):
        super().__init__()
        self.hidden_size = hidden_size
        self.epsilon = epsilon
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return RMSNormFunction.apply(input, self.weight, self.epsilon)

    def extra_repr(self) -> str:
        return f"hidden_size={self.hidden_size}, eps={self.epsilon}"


class AddRMSNormFunction(torch.autograd.Function):
    """(output, hidden) = (RMSNorm(input + residual) * weight, input + residual) in one kernel each way.

    The reference has no fused form: its users write `h = x + residual` and then call
    RMSNormFunction (megagemm/rmsnorm.py:18-48). Forward results are the same bits as that sequence;
    the backward adds the gradient arriving through `hidden` to the norm's input gradient before the
    one rounding.
    """

    @staticmethod
    def forward(ctx, input: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, epsilon: float = 1e-5):
        orig_shape = input.shape
        input_2d = input.view(-1, input.size(-1))
        residual_2d = residual.view(-1, residual.size(-1))
        output, hidden, inv_rms = rmsnorm_cuda_ops.add_rmsnorm_forward(input_2d, residual_2d, weight, epsilon)
        ctx.save_for_backward(hidden, weight, inv_rms)
        ctx.orig_shape = orig_shape
        ctx.set_materialize_grads(False)   # an output nobody differentiates arrives as None, not as zeros
        return output.view(orig_shape), hidden.view(orig_shape)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor, grad_hidden: torch.Tensor):
        hidden, weight, inv_rms = ctx.saved_tensors
        cols = hidden.size(-1)
        if grad_output is None and grad_hidden is None:
            return None, None, None, None
        if grad_output is None:
            grad_output = torch.zeros_like(hidden)
        grad_output_2d = grad_output.contiguous().view(-1, cols)
        if grad_hidden is None:
            grad_total, grad_weight = rmsnorm_cuda_ops.rmsnorm_backward(grad_output_2d, hidden, weight, inv_rms)
        else:
            grad_hidden_2d = grad_hidden.contiguous().view(-1, cols)
            grad_total, grad_weight, _ = rmsnorm_cuda_ops.add_rmsnorm_backward(grad_output_2d, grad_hidden_2d, hidden,
                                                                               weight, inv_rms)
        grad_total = grad_total.view(ctx.orig_shape)
        return grad_total, grad_total, grad_weight, None


class AddRMSNorm(RMSNorm):
    """RMSNorm that also performs the residual add in front of it: forward(input, residual) returns
    (RMSNorm(input + residual), input + residual). Same parameters and state dict as RMSNorm."""

    def forward(self, input: torch.Tensor, residual: torch.Tensor):  # type: ignore[override]
        return AddRMSNormFunction.apply(input, residual, self.weight, self.epsilon)
