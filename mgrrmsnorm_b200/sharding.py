"""Single-node multi-GPU forms of the two hot paths (one process per GPU, torch.distributed).

The reference has no distributed code at all; these wrappers add what its operators need to run
sharded while keeping its parameter layouts:

* RMSNorm shards by ROWS. Rows are independent (the forward grid is one CTA per row,
  src/rmsnorm_kernel.cu:531), so x, y, dy, dx and inv_rms stay local and the forward needs no
  collective. Only dW couples the shards: every rank all-reduces its fp32 column sum and then rounds
  once to the weight dtype, so results at 1/2/4/8 GPUs differ by fp32 reassociation only.
* The SwiGLU MLP is tensor-parallel. `w12.weight` is [2F, D] with the gate rows first and the value
  rows second (benchmark_swiglu.py:85-89), so rank r owns gate rows [rF/P, (r+1)F/P) AND value rows
  [F + rF/P, F + (r+1)F/P) -- two slices, stacked again as a local [2F/P, D] matrix of the same
  layout -- and columns [rF/P, (r+1)F/P) of `w3.weight` [D, F]. x is replicated; one all-reduce sums
  the partial outputs after w3 (forward) and one sums the partial dx (backward).

Index arithmetic and the collectives are plain torch and work on any backend (tests run them on gloo);
the compute they wrap is the CUDA library and needs a GPU.
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn

from . import rmsnorm_cuda_ops
from .swiglu import MegaGemmTriton


# ---------------------------------------------------------------------------------------------------
# index arithmetic
# ---------------------------------------------------------------------------------------------------

def row_shard(rows: int, world: int, rank: int) -> tuple[int, int]:
    """[r0, r1) of the contiguous row block rank `rank` owns; blocks differ by at most one row."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    base, extra = divmod(rows, world)
    r0 = rank * base + min(rank, extra)
    return r0, r0 + base + (1 if rank < extra else 0)


def tp_hidden_slice(hidden: int, world: int, rank: int) -> tuple[int, int]:
    """[f0, f1) of the hidden units rank `rank` owns. hidden must divide evenly."""
    if hidden % world != 0:
        raise ValueError(f"hidden size {hidden} is not divisible by the tensor-parallel size {world}")
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    per = hidden // world
    return rank * per, (rank + 1) * per


def tp_shard_w12(w12: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Local [2F/P, D] matrix: this rank's gate rows followed by its value rows."""
    hidden = w12.shape[0] // 2
    f0, f1 = tp_hidden_slice(hidden, world, rank)
    return torch.cat([w12[f0:f1], w12[hidden + f0:hidden + f1]], dim=0).contiguous()


def tp_shard_w3(w3: torch.Tensor, world: int, rank: int) -> torch.Tensor:
    """Local [D, F/P] matrix: this rank's columns of w3."""
    f0, f1 = tp_hidden_slice(w3.shape[1], world, rank)
    return w3[:, f0:f1].contiguous()


def tp_unshard_w12(shards: list[torch.Tensor]) -> torch.Tensor:
    """Inverse of tp_shard_w12 over all ranks: back to the reference layout [2F, D]."""
    per = shards[0].shape[0] // 2
    return torch.cat([s[:per] for s in shards] + [s[per:] for s in shards], dim=0)


def tp_unshard_w3(shards: list[torch.Tensor]) -> torch.Tensor:
    return torch.cat(shards, dim=1)


# ---------------------------------------------------------------------------------------------------
# collectives as autograd functions
# ---------------------------------------------------------------------------------------------------

class _ReduceForward(torch.autograd.Function):
    """all-reduce(SUM) in forward, identity in backward (sums the partial w3 outputs)."""

    @staticmethod
    def forward(ctx, t, group):
        out = t.contiguous().clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _ReduceBackward(torch.autograd.Function):
    """identity in forward, all-reduce(SUM) in backward (sums the partial dx of the replicated input)."""

    @staticmethod
    def forward(ctx, t, group):
        ctx.group = group
        return t.view_as(t)

    @staticmethod
    def backward(ctx, grad):
        out = grad.contiguous().clone()
        dist.all_reduce(out, op=dist.ReduceOp.SUM, group=ctx.group)
        return out, None


def allreduce_dw(dw_f32: torch.Tensor, out_dtype: torch.dtype, group=None) -> torch.Tensor:
    """Sums the per-rank fp32 dW partials in place over `group`, then rounds ONCE to `out_dtype`."""
    if dw_f32.dtype != torch.float32:
        raise TypeError("the cross-rank sum of dW is taken in fp32")
    dist.all_reduce(dw_f32, op=dist.ReduceOp.SUM, group=group)
    return dw_f32.to(out_dtype)


# ---------------------------------------------------------------------------------------------------
# row-sharded RMSNorm
# ---------------------------------------------------------------------------------------------------

class RowShardedRMSNormFunction(torch.autograd.Function):
    """RMSNormFunction for a rank that holds a row block: same forward; backward all-reduces dW."""

    @staticmethod
    def forward(ctx, input, weight, epsilon, group):
        orig_shape = input.shape
        input_2d = input.view(-1, input.size(-1))
        output, inv_rms = rmsnorm_cuda_ops.rmsnorm_forward(input_2d, weight, epsilon)
        ctx.save_for_backward(input_2d, weight, inv_rms)
        ctx.orig_shape = orig_shape
        ctx.group = group
        return output.view(orig_shape)

    @staticmethod
    def backward(ctx, grad_output):
        input_2d, weight, inv_rms = ctx.saved_tensors
        g2d = grad_output.contiguous().view(-1, grad_output.size(-1))
        grad_input, _, dw_f32 = rmsnorm_cuda_ops.rmsnorm_backward_full(g2d, input_2d, weight, inv_rms, want_dw_f32=True)
        grad_weight = allreduce_dw(dw_f32, weight.dtype, ctx.group)
        return grad_input.view(ctx.orig_shape), grad_weight, None, None


class RowShardedRMSNorm(nn.Module):
    """megagemm.RMSNorm whose input is this rank's row block of a larger batch; `weight` is replicated
    and its gradient is the sum over all ranks' rows."""

    def __init__(self, hidden_size: int, epsilon: float = 1e-5, group=None):
        super().__init__()
        self.hidden_size = hidden_size
        self.epsilon = epsilon
        self.group = group
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return RowShardedRMSNormFunction.apply(input, self.weight, self.epsilon, self.group)

    def extra_repr(self) -> str:
        return f"hidden_size={self.hidden_size}, eps={self.epsilon}, row-sharded"


# ---------------------------------------------------------------------------------------------------
# tensor-parallel SwiGLU MLP
# ---------------------------------------------------------------------------------------------------

# SMs kept free of GEMM CTAs while an all-reduce runs beside them (the GEMM kernels are persistent, one
# CTA per SM, and would otherwise leave the collective nowhere to run until they finish).
COMM_SMS = 16


class _OverlappedTPMLP(torch.autograd.Function):
    """One rank's share of the tensor-parallel MLP with its two all-reduces overlapped with GEMMs.

    Forward: the fused projection for all rows, then the w3 GEMM in `slabs` row slabs; the all-reduce of
    slab i (async, on NCCL's stream) runs while slab i+1 is multiplied. Backward: dx = dGV w12 first, its
    all-reduce in flight while dW12 = dGV^T x and dW3 = dy^T h are computed. The GEMMs launched while a
    collective is in flight leave COMM_SMS SMs free for it.
    """

    @staticmethod
    def forward(ctx, x, w12, w3, group, slabs):
        ops = rmsnorm_cuda_ops
        hidden = w3.shape[1]
        x2d = x.reshape(-1, x.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        m = x2d.shape[0]
        needs_grad = any(ctx.needs_input_grad[:3])
        if needs_grad:
            h, gv = ops.swiglu_fused_forward_save(x2d, w12, hidden)
        else:
            h, gv = ops.swiglu_fused_forward(x2d, w12, hidden), None
        y = torch.empty((m, w3.shape[0]), device=x.device, dtype=x.dtype)
        step = -(-m // slabs)
        step = -(-step // 256) * 256          # whole 256-row tiles per slab
        works = []
        with ops.gemm_sm_limit(COMM_SMS, x.device):
            for r0 in range(0, m, step):
                r1 = min(m, r0 + step)
                ops.linear_tn(h[r0:r1], w3, out=y[r0:r1])
                works.append(dist.all_reduce(y[r0:r1], op=dist.ReduceOp.SUM, group=group, async_op=True))
        for wk in works:
            wk.wait()
        if needs_grad:
            ctx.save_for_backward(x2d, w12, w3, h, gv)
        ctx.group = group
        ctx.x_shape = x.shape
        return y.view(x.shape[:-1] + (w3.shape[0],))

    @staticmethod
    def backward(ctx, grad_output):
        ops = rmsnorm_cuda_ops
        x2d, w12, w3, h, gv = ctx.saved_tensors
        hidden = w3.shape[1]
        dy = grad_output.reshape(-1, grad_output.shape[-1])
        if not dy.is_contiguous():
            dy = dy.contiguous()
        dgv = ops.swiglu_dh_dgv(dy, w3, gv, hidden)
        dx = ops.gemm(dgv, w12, False, True)
        work = dist.all_reduce(dx, op=dist.ReduceOp.SUM, group=ctx.group, async_op=True)   # x is replicated
        with ops.gemm_sm_limit(COMM_SMS, dy.device):
            dw12 = ops.gemm(dgv, x2d, True, True) if ctx.needs_input_grad[1] else None
            dw3 = ops.gemm(dy, h, True, True) if ctx.needs_input_grad[2] else None
        work.wait()
        return dx.view(ctx.x_shape), dw12, dw3, None, None


class TensorParallelSwiGLU(nn.Module):
    """MegaGemmTriton split over `group`: local `w12` [2F/P, D] and `w3` [D, F/P] (see module docstring).

    Build it from a full reference-layout module with `from_full`, or construct and load shards. The
    input is replicated on every rank; the output is the full [.., D] result on every rank.
    """

    def __init__(self, d_model: int, hidden: int, world: int, rank: int, group=None):
        super().__init__()
        f0, f1 = tp_hidden_slice(hidden, world, rank)
        self.hidden_full = hidden
        self.world, self.rank, self.group = world, rank, group
        self.overlap = True     # overlap the all-reduces with GEMMs (False: plain reduce after / before the local MLP)
        self.slabs = 4          # row slabs of the w3 GEMM whose all-reduces are pipelined
        self.local = MegaGemmTriton.__new__(MegaGemmTriton)
        nn.Module.__init__(self.local)
        self.local.hidden = f1 - f0
        self.local.w12 = nn.Linear(d_model, 2 * (f1 - f0), bias=False)
        self.local.w3 = nn.Linear(f1 - f0, d_model, bias=False)

    @classmethod
    def from_full(cls, full: MegaGemmTriton, world: int, rank: int, group=None) -> "TensorParallelSwiGLU":
        d_model = full.w12.in_features
        tp = cls(d_model, full.hidden, world, rank, group)
        tp = tp.to(device=full.w12.weight.device, dtype=full.w12.weight.dtype)
        with torch.no_grad():
            tp.local.w12.weight.copy_(tp_shard_w12(full.w12.weight, world, rank))
            tp.local.w3.weight.copy_(tp_shard_w3(full.w3.weight, world, rank))
        return tp

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        w12, w3 = self.local.w12.weight, self.local.w3.weight
        m = x.numel() // x.shape[-1] if x.numel() else 0
        if (self.overlap and x.is_cuda and x.dtype == w12.dtype and m > 0 and m % 8 == 0 and x.shape[-1] % 8 == 0
                and rmsnorm_cuda_ops._gemm_ok(w12, w3)):
            return _OverlappedTPMLP.apply(x, w12, w3, self.group, self.slabs)
        x = _ReduceBackward.apply(x, self.group)
        return _ReduceForward.apply(self.local(x), self.group)
