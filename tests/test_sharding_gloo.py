"""Host-side logic of the multi-GPU wrappers on CPU: index arithmetic, and the collectives run as two
gloo ranks. The CUDA compute they wrap is covered by the GPU tests; here the per-shard arithmetic is
done by the oracle so that the partitioning itself is what is checked."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mgrrmsnorm_b200 import sharding
from oracle import oracle


def test_row_shard_covers_all_rows_once():
    for rows in (0, 1, 7, 65536, 65537, 100003):
        for world in (1, 2, 3, 4, 8):
            spans = [sharding.row_shard(rows, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == rows
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert sharding.row_shard(65536, 8, 3) == (24576, 32768)
    with pytest.raises(ValueError):
        sharding.row_shard(8, 2, 2)


def test_tp_weight_shards_roundtrip_and_layout():
    d, f = 16, 24
    w12 = torch.arange(2 * f * d, dtype=torch.float32).view(2 * f, d)
    w3 = torch.arange(d * f, dtype=torch.float32).view(d, f)
    for world in (1, 2, 4):
        s12 = [sharding.tp_shard_w12(w12, world, r) for r in range(world)]
        s3 = [sharding.tp_shard_w3(w3, world, r) for r in range(world)]
        per = f // world
        for r in range(world):
            assert s12[r].shape == (2 * per, d) and s3[r].shape == (d, per)
            assert torch.equal(s12[r][:per], w12[r * per:(r + 1) * per])                 # gate rows of this rank
            assert torch.equal(s12[r][per:], w12[f + r * per:f + (r + 1) * per])         # value rows of this rank
        assert torch.equal(sharding.tp_unshard_w12(s12), w12)
        assert torch.equal(sharding.tp_unshard_w3(s3), w3)
    with pytest.raises(ValueError):
        sharding.tp_hidden_slice(10, 4, 0)
    # the configuration sizes: d_ff 28672 over 2/4/8 ranks
    assert [sharding.tp_hidden_slice(28672, p, p - 1) for p in (2, 4, 8)] == [(14336, 28672), (21504, 28672), (25088, 28672)]


def test_partial_sums_of_tp_shards_equal_the_full_mlp():
    """sum over ranks of w3_r( silu(x Wg_r^T) * (x Wv_r^T) ) == the unsharded MLP (oracle arithmetic)."""
    rng = np.random.default_rng(0)
    m, d, f = 6, 16, 24
    x = rng.standard_normal((m, d)).astype(np.float32)
    w12 = (rng.standard_normal((2 * f, d)) / 4).astype(np.float32)
    w3 = (rng.standard_normal((d, f)) / 4).astype(np.float32)
    dy = rng.standard_normal((m, d)).astype(np.float32)
    full = oracle.swiglu_mlp(x, w12, w3, dy=dy)
    for world in (2, 4):
        y = np.zeros((m, d))
        dx = np.zeros((m, d))
        dw12, dw3 = [], []
        for r in range(world):
            o = oracle.swiglu_mlp(x, sharding.tp_shard_w12(torch.from_numpy(w12), world, r).numpy(),
                                  sharding.tp_shard_w3(torch.from_numpy(w3), world, r).numpy(), dy=dy)
            y += o["y"]
            dx += o["dx"]
            dw12.append(torch.from_numpy(o["dw12"]))
            dw3.append(torch.from_numpy(o["dw3"]))
        np.testing.assert_allclose(y, full["y"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(dx, full["dx"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(sharding.tp_unshard_w12(dw12).numpy(), full["dw12"], rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(sharding.tp_unshard_w3(dw3).numpy(), full["dw3"], rtol=1e-12, atol=1e-12)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _gloo_worker(rank: int, world: int, port: int, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        rows, cols = 10, 8
        rng = np.random.default_rng(5)
        x = rng.standard_normal((rows, cols)).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
        dy = rng.standard_normal((rows, cols)).astype(np.float32)
        r0, r1 = sharding.row_shard(rows, world, rank)
        # each rank's fp32 dW partial over its own rows (oracle arithmetic), summed across ranks
        _, dw_local = oracle.rmsnorm_bwd(dy[r0:r1], x[r0:r1], w, 1e-6)
        dw = sharding.allreduce_dw(torch.from_numpy(dw_local.astype(np.float32)), torch.bfloat16)
        _, dw_full = oracle.rmsnorm_bwd(dy, x, w, 1e-6)
        ok_dw = dw.dtype == torch.bfloat16 and np.allclose(dw.float().numpy(), dw_full, rtol=1e-2, atol=1e-2)
        with pytest.raises(TypeError):
            sharding.allreduce_dw(torch.zeros(4, dtype=torch.float16), torch.float16)

        # The two legs of the benchmark take the cross-rank sum of dW through different helpers: the resident
        # loop through AsyncDwReduce (all-reduce + rounding off the compute stream), the host-tensor leg through
        # allreduce_dw on the pipeline's fp32 sum. Same shards in, same bits out: fp32 sum first, ONE rounding.
        # A sum of already-rounded partials (what the host leg once did) is a different number.
        big = 4096
        part = torch.from_numpy(np.random.default_rng(100 + rank).standard_normal(big).astype(np.float32) * 37.0)
        leg_host = sharding.allreduce_dw(part.clone(), torch.bfloat16)
        red = sharding.AsyncDwReduce("cpu")
        leg_resident = torch.empty(big, dtype=torch.bfloat16)
        scratch = part.clone()
        red.start(scratch, leg_resident)
        red.wait_for(scratch)
        red.drain()
        rounded_first = part.to(torch.bfloat16)
        dist.all_reduce(rounded_first)
        ok_dw = ok_dw and torch.equal(leg_host, leg_resident) and not torch.equal(leg_host, rounded_first)

        # forward-reduce / backward-reduce pair around a rank-local linear map
        t = torch.full((3,), float(rank + 1), requires_grad=True)
        a = sharding._ReduceBackward.apply(t, None)
        out = sharding._ReduceForward.apply(a * (rank + 1), None)
        out.sum().backward()
        total = sum((r + 1) ** 2 for r in range(world))
        ok_fwd = torch.allclose(out, torch.full((3,), float(total)))
        # d(out_sum)/dt on this rank is (rank+1); the backward all-reduce sums that over ranks
        ok_bwd = torch.allclose(t.grad, torch.full((3,), float(sum(r + 1 for r in range(world)))))
        q.put((rank, bool(ok_dw), bool(ok_fwd), bool(ok_bwd)))
    finally:
        dist.destroy_process_group()


def test_collectives_on_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] and r[2] and r[3] for r in results), results


# ---------------------------------------------------------------------------------------------------
# sequence-parallel MLP: slab cuts, the gathered row order and the collectives, on two gloo ranks.
# The kernels are replaced by a stand-in with the same signatures (fp64 torch on CPU), so what is
# checked here is everything around them: which rows are gathered where, which partial sums are
# scattered back to whom, and that the weight gradients cover every gathered row exactly once.
# ---------------------------------------------------------------------------------------------------

class _FakeKernels:
    """Signatures of the rmsnorm_cuda_ops entry points _SequenceParallelMLP calls; test code only."""

    class gemm_sm_limit:
        def __init__(self, reserve, device=None):
            pass

        def __enter__(self):
            return self

        def __exit__(self, *exc):
            return False

    @staticmethod
    def _act(gv, f):
        g, v = gv[:, :f], gv[:, f:]
        return torch.nn.functional.silu(g) * v

    @classmethod
    def swiglu_fused_forward_save(cls, x, w12, hidden, out_h=None, out_gv=None):
        gv = x @ w12.T
        out_gv.copy_(gv)
        out_h.copy_(cls._act(gv, hidden))
        return out_h, out_gv

    @classmethod
    def swiglu_fused_forward(cls, x, w12, hidden, out=None):
        out.copy_(cls._act(x @ w12.T, hidden))
        return out

    @staticmethod
    def linear_tn(a, b, out=None):
        return a @ b.T

    @staticmethod
    def swiglu_dh_dgv(dy, w3, gv, hidden, out=None):
        dh = dy @ w3
        g, v = gv[:, :hidden], gv[:, hidden:]
        s = torch.sigmoid(g)
        out.copy_(torch.cat([dh * v * s * (1 + g * (1 - s)), dh * g * s], dim=1))
        return out

    @staticmethod
    def gemm(a, b, a_mn_major=False, b_mn_major=False, out=None):
        a2 = a.T if a_mn_major else a
        b2 = b.T if b_mn_major else b
        return a2 @ b2.T


def test_slab_bounds():
    for rows, slabs in ((2048, 4), (16, 4), (8, 4), (24, 2), (4096, 3)):
        cuts = sharding.slab_bounds(rows, slabs)
        assert cuts[0][0] == 0 and cuts[-1][1] == rows and len(cuts) <= slabs
        assert all(a1 == b0 for (_, b0), (a1, _) in zip(cuts, cuts[1:]))
        assert all((b - a) % 8 == 0 for a, b in cuts)
    assert sharding.slab_bounds(0, 4) == []


def _sp_worker(rank: int, world: int, port: int, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sharding.rmsnorm_cuda_ops = _FakeKernels          # stand-in for the CUDA library (this process only)
        rng = np.random.default_rng(11)
        m_local, d, f = 24, 16, 8 * world
        m = m_local * world
        x = rng.standard_normal((m, d))
        w12 = rng.standard_normal((2 * f, d)) / 4
        w3 = rng.standard_normal((d, f)) / 4
        dy = rng.standard_normal((m, d))
        full = oracle.swiglu_mlp(x, w12, w3, dy=dy)
        r0, r1 = sharding.row_shard(m, world, rank)
        assert (r0, r1) == (rank * m_local, (rank + 1) * m_local)
        ok = True
        for slabs in (1, 2, 3):
            xl = torch.from_numpy(x[r0:r1].copy()).requires_grad_(True)
            w12l = sharding.tp_shard_w12(torch.from_numpy(w12), world, rank).requires_grad_(True)
            w3l = sharding.tp_shard_w3(torch.from_numpy(w3), world, rank).requires_grad_(True)
            out = sharding._SequenceParallelMLP.apply(xl, w12l, w3l, None, slabs)
            out.backward(torch.from_numpy(dy[r0:r1].copy()))
            ok &= np.allclose(out.detach().numpy(), full["y"][r0:r1], rtol=1e-10, atol=1e-10)
            ok &= np.allclose(xl.grad.numpy(), full["dx"][r0:r1], rtol=1e-10, atol=1e-10)
            f0, f1 = sharding.tp_hidden_slice(f, world, rank)
            want12 = np.concatenate([full["dw12"][f0:f1], full["dw12"][f + f0:f + f1]])
            ok &= np.allclose(w12l.grad.numpy(), want12, rtol=1e-10, atol=1e-10)
            ok &= np.allclose(w3l.grad.numpy(), full["dw3"][:, f0:f1], rtol=1e-10, atol=1e-10)
        # inference (no gradient wanted): the projection is not kept
        with torch.no_grad():
            out = sharding._SequenceParallelMLP.apply(torch.from_numpy(x[r0:r1].copy()), w12l.detach(), w3l.detach(), None, 2)
        ok &= np.allclose(out.numpy(), full["y"][r0:r1], rtol=1e-10, atol=1e-10)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_sequence_parallel_mlp_on_two_gloo_ranks():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_sp_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(r[0] for r in results) == [0, 1]
    assert all(r[1] for r in results), results


def test_sequence_parallel_module_checks_its_input():
    """Shape and dtype errors are raised before any collective or kernel is reached (no process group here)."""
    sp = sharding.SequenceParallelSwiGLU(64, 128, world=2, rank=1)
    assert tuple(sp.local.w12.weight.shape) == (128, 64) and tuple(sp.local.w3.weight.shape) == (64, 64)
    with pytest.raises(RuntimeError, match="multiples of 8"):
        sp(torch.zeros(12, 64))            # 12 rows: not a multiple of 8
    with pytest.raises(RuntimeError, match="multiples of 8"):
        sp(torch.zeros(0, 64))
    with pytest.raises(RuntimeError, match="share one dtype"):
        sp(torch.zeros(16, 64, dtype=torch.float16))
    with pytest.raises(ValueError):
        sharding.SequenceParallelSwiGLU(64, 100, world=3, rank=0)   # hidden not divisible by the group size


def test_index_arithmetic_properties():
    """row_shard blocks tile [0, rows) in rank order and differ by at most one row; slab_bounds tiles a rank's rows
    in multiples of eight; tensor-parallel weight shards put every hidden unit on exactly one rank."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=200, deadline=None)
    @given(rows=st.integers(0, 5000), world=st.integers(1, 16))
    def rows_tile(rows, world):
        blocks = [sharding.row_shard(rows, world, r) for r in range(world)]
        assert blocks[0][0] == 0 and blocks[-1][1] == rows
        assert all(b0[1] == b1[0] for b0, b1 in zip(blocks, blocks[1:]))
        sizes = [b - a for a, b in blocks]
        assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)

    @settings(max_examples=200, deadline=None)
    @given(k=st.integers(1, 600), slabs=st.integers(1, 12))
    def slabs_tile(k, slabs):
        rows = 8 * k
        cuts = sharding.slab_bounds(rows, slabs)
        assert 1 <= len(cuts) <= slabs and cuts[0][0] == 0 and cuts[-1][1] == rows
        assert all(c0[1] == c1[0] for c0, c1 in zip(cuts, cuts[1:]))
        assert all((b - a) % 8 == 0 and b > a for a, b in cuts)

    @settings(max_examples=50, deadline=None)
    @given(per=st.integers(1, 6), world=st.integers(1, 8), d=st.integers(1, 5))
    def shards_partition(per, world, d):
        f = per * world
        w12 = torch.arange(2 * f * d, dtype=torch.float32).view(2 * f, d)
        w3 = torch.arange(d * f, dtype=torch.float32).view(d, f)
        s12 = [sharding.tp_shard_w12(w12, world, r) for r in range(world)]
        s3 = [sharding.tp_shard_w3(w3, world, r) for r in range(world)]
        assert torch.equal(sharding.tp_unshard_w12(s12), w12) and torch.equal(sharding.tp_unshard_w3(s3), w3)
        assert all(s.shape == (2 * per, d) for s in s12) and all(s.shape == (d, per) for s in s3)

    rows_tile()
    slabs_tile()
    shards_partition()
