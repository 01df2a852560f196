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

import contextlib
import os

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


class AsyncDwReduce:
    """The cross-rank sum of the fp32 dW partials, taken OFF the compute stream.

    The all-reduce of a [H] fp32 vector is latency-bound (tens of microseconds for 32 KB) and nothing needs its
    result before the optimizer step, so it runs on a side stream beside whatever the compute stream does next
    (the next micro-batch's forward, the rest of the backward pass):

        red = AsyncDwReduce(device, group)
        ...backward kernel writes dw_f32 on the current stream...
        red.start(dw_f32, dw_out)       # all-reduce + the one rounding into dw_out (weight dtype), side stream
        ...more work on the current stream...
        red.wait_for(dw_f32)            # before dw_f32 is overwritten again
        red.drain()                     # before dw_out is read (optimizer step / end of a timed region)
    """

    def __init__(self, device=None, group=None, peer=None):
        # Host tensors (a CPU process group, as in the tests of the host logic) have no streams: the same sum and
        # rounding then run synchronously inside start().
        # `peer`: a PeerDwAllReduce of the same group; the sum is then that one kernel instead of an NCCL all-reduce and
        # a cast. The side stream has high priority: the compute stream's kernels are persistent and fill every SM, so
        # a collective queued beside them only gets CTAs as theirs retire, and with high priority it gets them before
        # the next compute kernel does (it needs 16 of them for a few microseconds).
        on_cpu = device is not None and torch.device(device).type == "cpu"
        self.side = None if on_cpu else torch.cuda.Stream(device, priority=-1)
        self.group = group
        self.peer = peer
        self.pending: dict[int, torch.cuda.Event] = {}

    def start(self, dw_f32: torch.Tensor, dw_out: torch.Tensor) -> None:
        if dw_f32.dtype != torch.float32:
            raise TypeError("the cross-rank sum of dW is taken in fp32")
        if self.side is None:
            dist.all_reduce(dw_f32, op=dist.ReduceOp.SUM, group=self.group)
            dw_out.copy_(dw_f32)
            return
        self.side.wait_stream(torch.cuda.current_stream(dw_f32.device))   # the partial has been produced
        # both tensors are used on the side stream: tell the caching allocator, so that freeing one of them on
        # the compute stream cannot hand its memory out again while the collective still runs
        dw_f32.record_stream(self.side)
        dw_out.record_stream(self.side)
        with torch.cuda.stream(self.side):
            if self.peer is not None:
                self.peer(dw_f32, dw_out)                                     # sum in rank order and the single rounding
            else:
                dist.all_reduce(dw_f32, op=dist.ReduceOp.SUM, group=self.group)
                dw_out.copy_(dw_f32)                                          # the single rounding
            ev = torch.cuda.Event()
            ev.record(self.side)
        self.pending[dw_f32.data_ptr()] = ev

    def wait_for(self, dw_f32: torch.Tensor) -> None:
        ev = self.pending.pop(dw_f32.data_ptr(), None)
        if ev is not None:
            torch.cuda.current_stream(dw_f32.device).wait_event(ev)

    def drain(self) -> None:
        if self.side is not None:
            torch.cuda.current_stream(self.side.device).wait_stream(self.side)
        self.pending.clear()


class PeerDwAllReduce:
    """The cross-rank fp32 sum of dW as ONE kernel per rank over NVLink peer memory (mgr_peer_allreduce_f32)
    instead of an NCCL all-reduce: for a 32 KB vector the collective is pure latency (18 us on 2-4 GPUs, 55 us on
    8, against a rank's 105 us forward+backward once 65 536 rows are split eight ways).

        red = PeerDwAllReduce(hidden, device, group)        # collective: every rank of the group constructs it
        ...backward kernel writes dw_f32 on the current stream...
        red(dw_f32, dw_out)                                 # current stream; dw_out = round(sum over ranks)

    Every rank stores its partial into every rank's buffer, waits until all partials have arrived in its own and
    adds them in rank order: the same bits on every rank. The buffers are torch symmetric memory (peer-mapped by
    the rendezvous); construction raises where that is not available, and callers fall back on allreduce_dw.
    Calls must be made by every rank, in the same order. The kernel's wait is bounded: a rank that never arrives
    shows up as MGR_ERR_DEVICE_TIMEOUT in rmsnorm_cuda_ops.device_status(), not as a hang."""

    def __init__(self, n_max: int, device, group=None):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _capi

        self.L = _capi.lib()
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.n_max = (int(n_max) + 3) // 4 * 4
        self.device = torch.device(device)
        nbytes = int(self.L.mgr_peer_allreduce_buffer_bytes(self.world, self.n_max))
        if nbytes == 0:
            raise RuntimeError("unsupported world size or vector length for the peer all-reduce")
        with torch.cuda.device(self.device):
            self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            self.buf.zero_()
            self.handle = symm_mem.rendezvous(self.buf, self.group.group_name if hasattr(self.group, "group_name") else self.group)
            ptrs = [int(p) for p in self.handle.buffer_ptrs]
            self.calls = torch.zeros(_capi.MGR_PEER_ALLREDUCE_CTAS, dtype=torch.int32, device=self.device)
            torch.cuda.synchronize(self.device)
        if len(ptrs) != self.world:
            raise RuntimeError("symmetric-memory rendezvous returned the wrong number of peers")
        self.ptrs = (ctypes.c_void_p * self.world)(*ptrs)
        dist.barrier(group=self.group)     # every rank's buffer is zeroed before anyone's first store can land in it

    def __call__(self, dw_f32: torch.Tensor, dw_out: torch.Tensor | None = None, out_f32: torch.Tensor | None = None) -> None:
        from . import _capi
        from .rmsnorm_cuda_ops import _DTYPES

        if dw_f32.dtype != torch.float32 or dw_f32.dim() != 1 or dw_f32.numel() > self.n_max or dw_f32.numel() % 4 != 0:
            raise RuntimeError("expected a float32 vector of a multiple of 4 elements, at most n_max")
        if dw_out is None and out_f32 is None:
            out_f32 = dw_f32
        code = _DTYPES[dw_out.dtype] if dw_out is not None else _capi.MGR_F32
        st = self.L.mgr_peer_allreduce_f32(self.ptrs, self.rank, self.world, dw_f32.data_ptr(),
                                           out_f32.data_ptr() if out_f32 is not None else None,
                                           dw_out.data_ptr() if dw_out is not None else None, code, dw_f32.numel(), self.n_max,
                                           self.calls.data_ptr(), torch.cuda.current_stream(self.device).cuda_stream)
        _capi.check("mgr_peer_allreduce_f32", st)


# ---------------------------------------------------------------------------------------------------
# row-sharded RMSNorm
# ---------------------------------------------------------------------------------------------------

class RowShardedRMSNormFunction(torch.autograd.Function):
    """RMSNormFunction for a rank that holds a row block: same forward; backward all-reduces dW."""

    @staticmethod
    def forward(ctx, input, weight, epsilon, group, peer=None):
        orig_shape = input.shape
        input_2d = input.view(-1, input.size(-1))
        output, inv_rms = rmsnorm_cuda_ops.rmsnorm_forward(input_2d, weight, epsilon)
        ctx.save_for_backward(input_2d, weight, inv_rms)
        ctx.orig_shape = orig_shape
        ctx.group = group
        ctx.peer = peer
        return output.view(orig_shape)

    @staticmethod
    def backward(ctx, grad_output):
        input_2d, weight, inv_rms = ctx.saved_tensors
        g2d = grad_output.contiguous().view(-1, grad_output.size(-1))
        grad_input, _, dw_f32 = rmsnorm_cuda_ops.rmsnorm_backward_full(g2d, input_2d, weight, inv_rms, want_dw_f32=True)
        if ctx.peer is not None:      # the library's peer-memory kernel: partials added in rank order, one rounding
            grad_weight = torch.empty_like(weight)
            ctx.peer(dw_f32, grad_weight)
        else:
            grad_weight = allreduce_dw(dw_f32, weight.dtype, ctx.group)
        return grad_input.view(ctx.orig_shape), grad_weight, None, None, None


class RowShardedRMSNorm(nn.Module):
    """megagemm.RMSNorm whose input is this rank's row block of a larger batch; `weight` is replicated
    and its gradient is the sum over all ranks' rows. `peer`: a PeerDwAllReduce of the same group (and at least
    hidden_size long); the sum is then taken by that kernel over NVLink peer memory instead of NCCL."""

    def __init__(self, hidden_size: int, epsilon: float = 1e-5, group=None, peer=None):
        super().__init__()
        self.hidden_size = hidden_size
        self.epsilon = epsilon
        self.group = group
        self.peer = peer
        self.weight = nn.Parameter(torch.ones(hidden_size))

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return RowShardedRMSNormFunction.apply(input, self.weight, self.epsilon, self.group, self.peer)

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


# ---------------------------------------------------------------------------------------------------
# sequence-parallel form of the pre-norm block: rows sharded outside the MLP, hidden units inside it
# ---------------------------------------------------------------------------------------------------

def slab_bounds(local_rows: int, slabs: int) -> list[tuple[int, int]]:
    """[a, b) row ranges that cut a rank's `local_rows` rows into at most `slabs` pieces, each a multiple of
    8 rows long except possibly the last. The same cut on every rank, since all ranks hold equally many rows."""
    if local_rows <= 0:
        return []
    step = -(-local_rows // max(1, slabs))
    step = -(-step // 8) * 8
    return [(a, min(local_rows, a + step)) for a in range(0, local_rows, step)]


# Which GEMMs of the sequence-parallel MLP leave COMM_SMS SMs to the collectives in flight beside them:
# "all" = every GEMM; "big" = per slab only the larger one (fused projection / dx GEMM); "small" = only the
# smaller one (w3 GEMM / dh-dGV kernel). A collective queued while an unrestricted persistent GEMM holds
# every SM starts when that GEMM ends. MGR_SP_LIMIT overrides (measurement aid).
SP_LIMIT = "all"


def _sp_limit(kind: str, device):
    mode = os.environ.get("MGR_SP_LIMIT", SP_LIMIT)
    on = mode == "all" or mode == kind
    return rmsnorm_cuda_ops.gemm_sm_limit(COMM_SMS, device) if on else contextlib.nullcontext()


class _SequenceParallelMLP(torch.autograd.Function):
    """One rank's share of the SwiGLU MLP when the tokens are sharded by rows outside it.

    The rank holds `m` rows of the (already normalised) input and F/P hidden units of the weights. The
    rows are cut into slabs; for slab s: all-gather that slab of every rank (P*m_s rows), fused
    projection + w3 GEMM on those rows with the local hidden units, reduce-scatter the partial result
    back so that each rank receives the sum for its own m_s rows. The MLP is row-wise independent, so
    the gathered rows are simply processed in the order they arrive (slab-major, then rank) and kept
    in that order for backward; no row is ever moved back into "global" order. The collectives of one
    slab run beside the GEMMs of its neighbours (async, on the communicator's stream; the GEMMs leave
    COMM_SMS SMs free).

    Backward mirrors it: all-gather the output gradient slab by slab, dh/dGV kernel and dx GEMM per slab,
    reduce-scatter each partial dx; the two weight-gradient GEMMs run once over all gathered rows.
    Against the all-reduce form this moves the same bytes but leaves the norm (and every other row-wise
    operation outside the MLP) with 1/P of the rows instead of a replicated copy.
    """

    @staticmethod
    def forward(ctx, x_local, w12, w3, group, slabs):
        ops = rmsnorm_cuda_ops
        world = dist.get_world_size(group)
        hidden = w3.shape[1]
        d_out = w3.shape[0]
        x2d = x_local.reshape(-1, x_local.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        m, d = x2d.shape
        cuts = slab_bounds(m, slabs)
        needs_grad = any(ctx.needs_input_grad[:3])
        xg = x2d.new_empty((world * m, d))                      # gathered rows, slab-major then rank
        h = x2d.new_empty((world * m, hidden))
        gv = x2d.new_empty((world * m, 2 * hidden)) if needs_grad else None
        out = x2d.new_empty((m, d_out))
        gathers = [dist.all_gather_into_tensor(xg[world * a:world * b], x2d[a:b], group=group, async_op=True)
                   for a, b in cuts]
        pending = []
        for (a, b), wk in zip(cuts, gathers):
            wk.wait()
            ga, gb = world * a, world * b
            with _sp_limit("big", x2d.device):
                if needs_grad:
                    ops.swiglu_fused_forward_save(xg[ga:gb], w12, hidden, out_h=h[ga:gb], out_gv=gv[ga:gb])
                else:
                    ops.swiglu_fused_forward(xg[ga:gb], w12, hidden, out=h[ga:gb])
            with _sp_limit("small", x2d.device):
                part = ops.linear_tn(h[ga:gb], w3)
            pending.append((dist.reduce_scatter_tensor(out[a:b], part, op=dist.ReduceOp.SUM, group=group, async_op=True), part))
        for wk, _ in pending:
            wk.wait()
        if needs_grad:
            ctx.save_for_backward(xg, w12, w3, h, gv)
        ctx.group, ctx.cuts, ctx.world = group, cuts, world
        ctx.x_shape = x_local.shape
        return out.view(x_local.shape[:-1] + (d_out,))

    @staticmethod
    def backward(ctx, grad_output):
        ops = rmsnorm_cuda_ops
        xg, w12, w3, h, gv = ctx.saved_tensors
        world, cuts, group = ctx.world, ctx.cuts, ctx.group
        hidden = w3.shape[1]
        dy = grad_output.reshape(-1, grad_output.shape[-1])
        if not dy.is_contiguous():
            dy = dy.contiguous()
        m = dy.shape[0]
        dyg = dy.new_empty((world * m, dy.shape[1]))
        dgv = torch.empty_like(gv)
        dx = dy.new_empty((m, xg.shape[1]))
        gathers = [dist.all_gather_into_tensor(dyg[world * a:world * b], dy[a:b], group=group, async_op=True)
                   for a, b in cuts]
        pending = []
        for (a, b), wk in zip(cuts, gathers):
            wk.wait()
            ga, gb = world * a, world * b
            with _sp_limit("small", dy.device):
                ops.swiglu_dh_dgv(dyg[ga:gb], w3, gv[ga:gb], hidden, out=dgv[ga:gb])
            with _sp_limit("big", dy.device):
                part = ops.gemm(dgv[ga:gb], w12, False, True)
            pending.append((dist.reduce_scatter_tensor(dx[a:b], part, op=dist.ReduceOp.SUM, group=group, async_op=True), part))
        with ops.gemm_sm_limit(COMM_SMS, dy.device):      # the last reduce-scatter is in flight beside this one
            dw12 = ops.gemm(dgv, xg, True, True) if ctx.needs_input_grad[1] else None
        dw3 = ops.gemm(dyg, h, True, True) if ctx.needs_input_grad[2] else None
        for wk, _ in pending:
            wk.wait()
        return dx.view(ctx.x_shape), dw12, dw3, None, None


class SequenceParallelSwiGLU(TensorParallelSwiGLU):
    """TensorParallelSwiGLU whose input and output are this rank's ROW block [.., m, D] of the batch
    (every rank the same number of rows) instead of replicated tensors. Same weight shards, same
    `from_full`. Put a RowShardedRMSNorm in front of it for the pre-norm block: the norm then touches
    1/P of the rows, and its dW is the all-reduced fp32 sum."""

    def forward(self, x_local: torch.Tensor) -> torch.Tensor:
        w12, w3 = self.local.w12.weight, self.local.w3.weight
        m = x_local.numel() // x_local.shape[-1] if x_local.numel() else 0
        if m == 0 or m % 8 != 0 or x_local.shape[-1] % 8 != 0:
            raise RuntimeError("sequence-parallel MLP needs a non-empty row block whose row count and width are multiples of 8")
        if x_local.dtype != w12.dtype:
            raise RuntimeError("input and weights must share one dtype")
        return _SequenceParallelMLP.apply(x_local, w12, w3, self.group, self.slabs)
