"""Row-sharded RMSNorm, tensor-parallel SwiGLU and the sequence-parallel pre-norm block on two real GPUs
(NCCL), against the single-GPU result of the same library. Skipped with fewer than two devices. Ranks are child processes; in
the first test they meet only in collectives between kernels, with NVLS switched off. The second test runs the library's
own peer-memory sum of dW, whose kernel waits for its peers with a bound of about a second and reports a timeout through
the status word; no rank leaves early and nothing is made to time out."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from mgrrmsnorm_b200 import MegaGemmTriton, RMSNorm, sharding

        # ---- row-sharded RMSNorm: 2 x 1500 rows of hidden 4096, bf16
        g = torch.Generator().manual_seed(1234)
        rows, cols = 3000, 4096
        x = (2 ** 0.5 * torch.randn(rows, cols, generator=g)).bfloat16()
        w = (1 + 0.1 * torch.randn(cols, generator=g)).bfloat16()
        dy = torch.randn(rows, cols, generator=g).bfloat16()
        full = RMSNorm(cols, epsilon=1e-6).to(dev).bfloat16()
        shard = sharding.RowShardedRMSNorm(cols, epsilon=1e-6).to(dev).bfloat16()
        with torch.no_grad():
            full.weight.copy_(w.to(dev))
            shard.weight.copy_(w.to(dev))
        xf = x.to(dev).requires_grad_(True)
        yf = full(xf)
        yf.backward(dy.to(dev))
        r0, r1 = sharding.row_shard(rows, world, rank)
        xs = x[r0:r1].to(dev).requires_grad_(True)
        ys = shard(xs)
        ys.backward(dy[r0:r1].to(dev))
        ok_rows = torch.equal(ys, yf[r0:r1]) and torch.equal(xs.grad, xf.grad[r0:r1])
        # fp32 partial sums are added across ranks before the single rounding: at most one bf16 ulp from
        # the one-GPU result (a different fp32 summation order next to a rounding boundary). Columns whose sum
        # nearly cancels (|dW| << the terms' size) carry the fp32 summation error itself, hence the absolute floor.
        dws, dwf = shard.weight.grad.float(), full.weight.grad.float()
        ulp = torch.maximum(dws.abs(), dwf.abs()) * 2.0 ** -7 + 1e-4
        worst = int(((dws - dwf).abs() - ulp).argmax())
        ok_dw = bool(((dws - dwf).abs() <= ulp).all()) and float((dws != dwf).float().mean()) < 0.05
        if not ok_dw:
            ok_dw = (f"dw differs: column {worst}: {float(dws[worst])!r} vs {float(dwf[worst])!r}; "
                     f"{float((dws != dwf).float().mean()):.4f} of the columns differ")

        # the same sum taken off the compute stream (AsyncDwReduce): identical bits to the synchronous path
        import rmsnorm_cuda_ops as ops

        _, inv_s = ops.rmsnorm_forward(xs.detach(), shard.weight.detach(), 1e-6)
        red = sharding.AsyncDwReduce(dev)
        outs_async = []
        for _ in range(3):                                  # the partial buffer is reused: wait_for orders the reuse
            _, _, dw32 = ops.rmsnorm_backward_full(dy[r0:r1].to(dev), xs.detach(), shard.weight.detach(), inv_s, want_dw_f32=True)
            dw_out = torch.empty_like(shard.weight)
            red.start(dw32, dw_out)
            red.wait_for(dw32)
            outs_async.append(dw_out)
        red.drain()
        torch.cuda.synchronize()
        if ok_dw is True and not all(torch.equal(o, shard.weight.grad) for o in outs_async):
            ok_dw = "AsyncDwReduce result differs from the synchronous all-reduce"

        # ---- tensor-parallel MLP: d_model 512, hidden 1024 split over 2 ranks, fp16
        torch.manual_seed(7)
        mlp = MegaGemmTriton(512, multiple_of=256, hidden_multiple=2.0).to(dev).half()
        for p in mlp.parameters():            # same weights on every rank
            dist.broadcast(p.data, src=0)
        tp = sharding.TensorParallelSwiGLU.from_full(mlp, world, rank)
        xm = torch.randn(256, 512, generator=g).half()
        dym = torch.randn(256, 512, generator=g).half()
        a = xm.to(dev).requires_grad_(True)
        ya = mlp(a)
        ya.backward(dym.to(dev))
        f0, f1 = sharding.tp_hidden_slice(mlp.hidden, world, rank)
        tol = 2e-2
        gw12 = torch.cat([mlp.w12.weight.grad[f0:f1], mlp.w12.weight.grad[mlp.hidden + f0:mlp.hidden + f1]])
        ok_y = ok_dx = ok_w12 = ok_w3 = True
        outs = []
        for overlap in (False, True):       # plain reduce around the local MLP, and all-reduces overlapped with GEMMs
            tp.overlap = overlap
            tp.slabs = 2
            tp.local.w12.weight.grad = None
            tp.local.w3.weight.grad = None
            b = xm.to(dev).requires_grad_(True)
            yb = tp(b)
            yb.backward(dym.to(dev))
            ok_y &= float((ya.float() - yb.float()).abs().max()) < tol
            ok_dx &= float((a.grad.float() - b.grad.float()).abs().max()) < tol
            ok_w12 &= float((gw12.float() - tp.local.w12.weight.grad.float()).abs().max()) < 5e-2
            ok_w3 &= float((mlp.w3.weight.grad[:, f0:f1].float() - tp.local.w3.weight.grad.float()).abs().max()) < 5e-2
            outs.append((yb.detach().clone(), b.grad.clone()))
        # the two schedules run the same kernels on the same data: identical results
        ok_y &= torch.equal(outs[0][0], outs[1][0])
        ok_dx &= torch.equal(outs[0][1], outs[1][1])

        # ---- sequence-parallel pre-norm block: rows sharded outside the MLP (norm on 1/P of the rows, all-gather,
        # MLP on the local hidden units, reduce-scatter), against norm -> MLP on one GPU with the same weights
        norm1 = RMSNorm(512, epsilon=1e-6).to(dev).half()
        with torch.no_grad():
            norm1.weight.copy_((1 + 0.1 * torch.randn(512, generator=g)).half().to(dev))
        mlp.zero_grad()
        a = xm.to(dev).requires_grad_(True)
        ya = mlp(norm1(a))
        ya.backward(dym.to(dev))
        gw12 = torch.cat([mlp.w12.weight.grad[f0:f1], mlp.w12.weight.grad[mlp.hidden + f0:mlp.hidden + f1]])
        sp = sharding.SequenceParallelSwiGLU.from_full(mlp, world, rank)
        norm_s = sharding.RowShardedRMSNorm(512, epsilon=1e-6).to(dev).half()
        with torch.no_grad():
            norm_s.weight.copy_(norm1.weight)
        r0, r1 = sharding.row_shard(xm.shape[0], world, rank)
        sp_bad = []          # names of the checks that failed, for the assertion message

        def close(name, got, want, rel):
            # |got - want| <= rel * max|want|: the two paths round their fp16 intermediates at different points
            # (partial sums are rounded before the cross-rank sum), so the error scales with the values' size
            err = float((got.float() - want.float()).abs().max())
            if not err <= rel * max(float(want.float().abs().max()), 1.0):
                sp_bad.append(f"{name}: err {err:.4g} vs max {float(want.float().abs().max()):.4g}")

        sp_outs = []
        for slabs in (1, 3):
            sp.slabs = slabs
            sp.zero_grad()
            norm_s.zero_grad()
            b = xm[r0:r1].to(dev).requires_grad_(True)
            yb = sp(norm_s(b))
            yb.backward(dym[r0:r1].to(dev))
            if tuple(yb.shape) != (r1 - r0, 512):
                sp_bad.append("shape")
            close(f"y/{slabs}", yb, ya[r0:r1], 2e-2)
            close(f"dx/{slabs}", b.grad, a.grad[r0:r1], 2e-2)
            close(f"dw12/{slabs}", sp.local.w12.weight.grad, gw12, 2e-2)
            close(f"dw3/{slabs}", sp.local.w3.weight.grad, mlp.w3.weight.grad[:, f0:f1], 2e-2)
            close(f"dw_norm/{slabs}", norm_s.weight.grad, norm1.weight.grad, 2e-2)
            sp_outs.append((yb.detach().clone(), b.grad.clone()))
        # forward rows do not depend on how they are cut into slabs (each row is one independent GEMM row)
        if not torch.equal(sp_outs[0][0], sp_outs[1][0]):
            sp_bad.append("forward differs between 1 and 3 slabs: max %.4g" % float((sp_outs[0][0].float() - sp_outs[1][0].float()).abs().max()))
        ok_sp = "; ".join(sp_bad) if sp_bad else True
        torch.cuda.synchronize()
        q.put((rank, ok_rows, ok_dw, ok_y, ok_dx, ok_w12, ok_w3, ok_sp))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_sharded_paths_on_two_gpus(built_lib):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for r in results:
        assert all(v is True or v == 1 for v in r[1:]), f"rank {r[0]}: rows/dw/y/dx/dw12/dw3/sequence-parallel = {r[1:]}"


def _peer_worker(rank: int, world: int, port: int, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import rmsnorm_cuda_ops as ops
        from mgrrmsnorm_b200 import sharding

        n = 8192
        try:
            red = sharding.PeerDwAllReduce(n, dev)
        except Exception as e:  # noqa: BLE001  (no symmetric memory on this machine: nothing to test)
            q.put((rank, "skip", repr(e)[:200]))
            return
        g = torch.Generator(device=dev).manual_seed(50 + rank)
        bad = []
        for it, m in enumerate((8192, 8192, 4096, 8, 8192, 2560)):          # shorter vectors reuse the same buffers
            part = torch.randn(m, device=dev, generator=g) * (10.0 ** (it % 3))
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            want = parts[0].clone()
            for p_ in parts[1:]:
                want += p_                                                    # rank order, as the kernel adds them
            out32 = torch.empty_like(part)
            out16 = torch.empty(m, device=dev, dtype=torch.bfloat16)
            red(part, out16, out32)
            torch.cuda.synchronize()
            if not torch.equal(out32, want):
                bad.append(f"call {it}: fp32 sum differs (max {float((out32 - want).abs().max()):.3g})")
            if not torch.equal(out16, want.to(torch.bfloat16)):
                bad.append(f"call {it}: rounded sum differs")
        # behind the side-stream helper: same bits, and the partial buffer may be reused after wait_for
        helper = sharding.AsyncDwReduce(dev, peer=red)
        part = torch.randn(n, device=dev, generator=g)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        want = sum(parts[1:], parts[0].clone())
        outs = []
        for _ in range(3):
            o = torch.empty(n, device=dev, dtype=torch.float16)
            helper.start(part, o)
            helper.wait_for(part)
            outs.append(o)
        helper.drain()
        torch.cuda.synchronize()
        if not all(torch.equal(o, want.to(torch.float16)) for o in outs):
            bad.append("AsyncDwReduce(peer=...) differs from the rank-ordered sum")
        # inside the row-sharded module: dW = the one rounding of the rank-ordered sum of the ranks' fp32 partials
        gen = torch.Generator().manual_seed(9)
        rows, cols = 1000, 4096
        x = torch.randn(rows, cols, generator=gen).bfloat16()
        dy = torch.randn(rows, cols, generator=gen).bfloat16()
        r0, r1 = sharding.row_shard(rows, world, rank)
        mod = sharding.RowShardedRMSNorm(cols, epsilon=1e-6, peer=red).to(dev).bfloat16()
        xs = x[r0:r1].to(dev).requires_grad_(True)
        mod(xs).backward(dy[r0:r1].to(dev))
        _, inv = ops.rmsnorm_forward(xs.detach(), mod.weight.detach(), 1e-6)
        _, _, part = ops.rmsnorm_backward_full(dy[r0:r1].to(dev), xs.detach(), mod.weight.detach(), inv, want_dw_f32=True)
        parts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(parts, part)
        want = sum(parts[1:], parts[0].clone()).to(torch.bfloat16)
        torch.cuda.synchronize()
        if not torch.equal(mod.weight.grad, want):
            bad.append("RowShardedRMSNorm(peer=...) weight gradient differs from the rank-ordered sum")
        try:
            ops.device_status()
        except Exception as e:  # noqa: BLE001
            bad.append(f"device status: {e}")
        q.put((rank, "; ".join(bad) if bad else True, ""))
    finally:
        dist.barrier()
        dist.destroy_process_group()


def test_peer_memory_dw_sum_on_two_gpus(built_lib):
    """mgr_peer_allreduce_f32 through sharding.PeerDwAllReduce: every rank gets the partials added in rank order
    (bit-equal to that sum computed with torch on gathered partials), the rounded output is its one rounding,
    vectors shorter than the buffers' capacity work, and the side-stream helper gives the same bits."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_peer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    if any(r[1] == "skip" for r in results):
        pytest.skip(f"symmetric memory unavailable: {results[0][2]}")
    for r in results:
        assert r[1] is True, f"rank {r[0]}: {r[1]}"
