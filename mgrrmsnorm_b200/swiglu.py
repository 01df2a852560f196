"""SwiGLU MLP module and activation Function: the host-side mirror of megagemm/swiglu.py.

Same class names, constructor arguments, attributes (`w12`, `w3`, `hidden`) and parameter layout as
the reference (megagemm/swiglu.py:86-172): `w12.weight` is [2*hidden, d_model] with the gate rows
first and the value rows second (benchmark_swiglu.py:85-89), `w3.weight` is [d_model, hidden], no
biases -- so the reference's state dicts load unchanged. The Triton kernels are gone: the
activation runs in libmgr_b200.so.
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.autograd import Function

from . import rmsnorm_cuda_ops


class MegaGemmFunction(Function):
    """silu(gate) * value on a projected tensor [..., 2*hidden] (megagemm/swiglu.py:86-131)."""

    @staticmethod
    def forward(ctx, w12_out: torch.Tensor, hidden_dim: int):
        w12_out = w12_out.contiguous()
        x_flat = w12_out.view(-1, 2 * hidden_dim)
        out_flat = rmsnorm_cuda_ops.swiglu_act_forward(x_flat, hidden_dim)
        ctx.save_for_backward(w12_out)
        ctx.hidden_dim = hidden_dim
        return out_flat.view(w12_out.shape[:-1] + (hidden_dim,))

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        (w12_out,) = ctx.saved_tensors
        hidden_dim = ctx.hidden_dim
        grad_out_flat = grad_output.contiguous().view(-1, hidden_dim)
        x_flat = w12_out.contiguous().view(-1, 2 * hidden_dim)
        grad_input_flat = rmsnorm_cuda_ops.swiglu_act_backward(grad_out_flat, x_flat, hidden_dim)
        return grad_input_flat.view(w12_out.shape), None


def _recompute_projection() -> bool:
    """MGR_MLP_RECOMPUTE=1 trades one more projection GEMM in backward for not keeping [M, 2*hidden]."""
    import os

    return os.environ.get("MGR_MLP_RECOMPUTE", "0") not in ("", "0")


class SwiGLUMLPFunction(Function):
    """The whole MLP, y = w3(silu(x w1^T) * (x w2^T)), on the tensor-core kernels.

    Forward: one fused kernel produces h = silu(gate) * value straight from the fp32 accumulators, then
    the w3 GEMM. Without autograd (inference) the [M, 2*hidden] projection the reference materialises
    between megagemm/swiglu.py:167 and :168 never exists. With autograd it is written once by the same
    kernel and kept for backward, as the reference keeps w12_out (:98) -- unless MGR_MLP_RECOMPUTE=1,
    in which case backward recomputes it tile by tile instead.
    Backward follows the reference's autograd graph (Linear(w3) -> MegaGemmFunction -> Linear(w12)) in
    four GEMM launches: dW3 = dy^T h; [d_gate | d_val] as the epilogue of dh = dy w3 (dh itself is
    never stored); dx = dGV w12; dW12 = dGV^T x. No operand is transposed in memory.
    """

    @staticmethod
    def forward(ctx, x: torch.Tensor, w12: torch.Tensor, w3: torch.Tensor):
        ops = rmsnorm_cuda_ops
        hidden = w3.shape[1]
        x2d = x.reshape(-1, x.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        needs_grad = any(ctx.needs_input_grad)
        keep = needs_grad and not _recompute_projection() and x2d.shape[0] % 8 == 0
        if keep:
            h, gv = ops.swiglu_fused_forward_save(x2d, w12, hidden)
        else:
            h, gv = ops.swiglu_fused_forward(x2d, w12, hidden), None
        y = ops.linear_tn(h, w3)
        if needs_grad:
            ctx.save_for_backward(x2d, w12, w3, h, *([gv] if keep else []))
        ctx.kept = keep
        ctx.x_shape = x.shape
        return y.view(x.shape[:-1] + (w3.shape[0],))

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        ops = rmsnorm_cuda_ops
        x2d, w12, w3, h = ctx.saved_tensors[:4]
        hidden = w3.shape[1]
        dy = grad_output.reshape(-1, grad_output.shape[-1])
        if not dy.is_contiguous():
            dy = dy.contiguous()
        m = x2d.shape[0]
        if m % 8 != 0:
            # dW = (.)^T (.) contracts over the M rows; the tensor-core kernel wants that length to be a
            # multiple of 8. Ragged batches keep the library GEMMs for backward.
            dh = torch.matmul(dy, w3)
            dw3 = torch.matmul(dy.t(), h) if ctx.needs_input_grad[2] else None
            dgv = ops.swiglu_act_backward(dh, torch.nn.functional.linear(x2d, w12), hidden)
            dx = torch.matmul(dgv, w12).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
            dw12 = torch.matmul(dgv.t(), x2d) if ctx.needs_input_grad[1] else None
            return dx, dw12, dw3
        dw3 = ops.gemm(dy, h, True, True) if ctx.needs_input_grad[2] else None        # dy^T h     -> [D, F]
        if ctx.kept:
            dgv = ops.swiglu_dh_dgv(dy, w3, ctx.saved_tensors[4], hidden)    # dh = dy w3, fused        -> [M, 2F]
        else:
            dh = ops.gemm(dy, w3, False, True)                               # dy [M,D] x w3 [D,F]      -> [M, F]
            dgv = ops.swiglu_fused_backward(dh, x2d, w12, hidden)            # projection recomputed    -> [M, 2F]
        dx = ops.gemm(dgv, w12, False, True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None   # -> [M, D]
        dw12 = ops.gemm(dgv, x2d, True, True) if ctx.needs_input_grad[1] else None    # dgv^T x   -> [2F, D]
        return dx, dw12, dw3


class MegaGemmTriton(nn.Module):
    """SwiGLU MLP: y = w3( silu(x w1^T) * (x w2^T) ), w1|w2 stacked in `w12`.

    Args (as megagemm/swiglu.py:156): d_model, multiple_of=256, hidden_multiple=5/3. `hidden` is
    int(d_model*hidden_multiple) rounded up to a multiple of `multiple_of` (:158-160). The class keeps
    the reference's name although nothing here uses Triton.
    """

    def __init__(self, d_model: int, multiple_of: int = 256, hidden_multiple: float = 5 / 3):
        super().__init__()
        hidden = int(d_model * hidden_multiple)
        hidden = multiple_of * ((hidden + multiple_of - 1) // multiple_of)
        self.hidden = hidden
        self.w12 = nn.Linear(d_model, 2 * hidden, bias=False)
        self.w3 = nn.Linear(hidden, d_model, bias=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w12, w3 = self.w12.weight, self.w3.weight
        if x.is_cuda and x.dtype == w12.dtype and x.numel() > 0 and x.shape[-1] % 8 == 0 and \
                rmsnorm_cuda_ops._gemm_ok(w12, w3):
            return SwiGLUMLPFunction.apply(x, w12, w3)
        # fp32 modules and shapes the tensor-core kernels do not take keep the reference's own
        # structure (megagemm/swiglu.py:166-169): library GEMM, activation kernel, library GEMM.
        w12_out = self.w12(x)
        hidden = MegaGemmFunction.apply(w12_out, self.hidden)
        return self.w3(hidden)

    def extra_repr(self) -> str:
        return f"d_model={self.w12.in_features}, hidden={self.hidden} (sm_100a)"


class PreNormSwiGLU(nn.Module):
    """The pre-norm MLP block y = mlp(norm(x)) with the norm folded into the projection at inference time.

    A user of the reference writes `mlp(norm(x))`: RMSNorm writes the normalised [M, D] tensor
    (megagemm/rmsnorm.py:74-75) and `self.w12` reads it back (megagemm/swiglu.py:167). Here, when no gradient
    is wanted, that tensor never exists: since norm(x)[r, k] = x[r, k] * inv_rms[r] * w[k],

        w12(norm(x))[r, n] = inv_rms[r] * sum_k x[r, k] * (w[k] * w12[n, k]),

    so the norm weight is folded into the columns of w12 once (kept until either parameter changes), one
    light kernel reads x for the row scales (rms_inv), and the projection kernel multiplies its accumulator
    rows by inv_rms[r] before the activation. With gradients enabled the block runs as the two modules it is
    made of (the folded weight would have to be rebuilt every step, which costs more than it saves).

    Results differ from the two-step path by rounding only: there norm(x) is rounded to the tensor dtype
    before the GEMM, here w * w12 is.
    """

    def __init__(self, norm: nn.Module, mlp: MegaGemmTriton):
        super().__init__()
        self.norm = norm
        self.mlp = mlp
        self._folded = None
        self._folded_key = None

    def folded_w12(self) -> torch.Tensor:
        w, w12 = self.norm.weight, self.mlp.w12.weight
        key = (w.data_ptr(), w._version, w12.data_ptr(), w12._version, w12.dtype, w12.device)
        if self._folded is None or self._folded_key != key:
            with torch.no_grad():
                self._folded = (w12.float() * w.float().unsqueeze(0)).to(w12.dtype).contiguous()
            self._folded_key = key
        return self._folded

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w12, w3 = self.mlp.w12.weight, self.mlp.w3.weight
        fused = (not torch.is_grad_enabled() and x.is_cuda and x.dtype == w12.dtype and x.numel() > 0
                 and x.shape[-1] % 8 == 0 and x.is_contiguous() and rmsnorm_cuda_ops._gemm_ok(w12, w3)
                 and self.norm.weight.dtype == w12.dtype)
        if not fused:
            return self.mlp(self.norm(x))
        x2d = x.view(-1, x.shape[-1])
        inv = rmsnorm_cuda_ops.rms_inv(x2d, self.norm.epsilon)
        h = rmsnorm_cuda_ops.swiglu_fused_forward(x2d, self.folded_w12(), self.mlp.hidden, row_scale=inv)
        y = rmsnorm_cuda_ops.linear_tn(h, w3)
        return y.view(x.shape[:-1] + (w3.shape[0],))
