"""The compiled `rmsnorm_cuda_ops` extension on the GPU: every entry point against the ctypes route (same
C ABI, so the same bits) and the RMSNorm set against the oracle; plus the per-call host cost of both."""
import time

import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import TORCH_DTYPES, assert_matches_truth, seeded_rmsnorm_inputs, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def routes(built_lib):
    from mgrrmsnorm_b200 import build

    build.build_binding()
    import mgrrmsnorm_b200.rmsnorm_cuda_ops as ops
    from mgrrmsnorm_b200.pybind import rmsnorm_cuda_ops as ext

    return ext, ops.ctypes_impl


def same(a, b):
    if a is None or b is None:
        return a is None and b is None
    return torch.equal(a, b)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("rows,cols", [(1, 2), (7, 1000), (129, 128), (300, 4096), (2100, 8192), (40, 16384), (77, 2560)])
def test_rmsnorm_through_the_extension(routes, dtype, rows, cols):
    ext, py = routes
    x, w, dy = seeded_rmsnorm_inputs(rows, cols, dtype, rows * 3 + cols)
    xd, wd, dyd = x.cuda(), w.cuda(), dy.cuda()
    y, inv = ext.rmsnorm_forward(xd, wd, 1e-6)
    dx, dw, dw32 = ext.rmsnorm_backward_full(dyd, xd, wd, inv, True)
    dx2, dw2 = ext.rmsnorm_backward(dyd, xd, wd, inv)
    torch.cuda.synchronize()
    ty, tinv = oracle.rmsnorm_fwd(to_np(x), to_np(w), 1e-6)
    tdx, tdw = oracle.rmsnorm_bwd(to_np(dy), to_np(x), to_np(w), 1e-6)
    assert_matches_truth(y, ty, dtype, "y")
    assert_matches_truth(inv, tinv, "f32", "inv_rms")
    assert_matches_truth(dx, tdx, dtype, "dx")
    assert_matches_truth(dw32, tdw, "f32", "dw_f32", slack=4.0)
    assert torch.equal(dw, dw32.to(dw.dtype)) and torch.equal(dx, dx2) and torch.equal(dw, dw2)
    py_y, py_inv = py["rmsnorm_forward"](xd, wd, 1e-6)
    py_dx, py_dw, py_dw32 = py["rmsnorm_backward_full"](dyd, xd, wd, inv, want_dw_f32=True)
    assert all(same(a, b) for a, b in ((y, py_y), (inv, py_inv), (dx, py_dx), (dw, py_dw), (dw32, py_dw32)))


def test_every_other_entry_point_gives_the_ctypes_route_bits(routes):
    ext, py = routes
    g = torch.Generator().manual_seed(77)
    td = torch.bfloat16
    m, d, f = 264, 256, 384
    x = torch.randn(m, d, generator=g).to(td).cuda()
    res = torch.randn(m, d, generator=g).to(td).cuda()
    wn = (1 + 0.1 * torch.randn(d, generator=g)).to(td).cuda()
    w12 = (torch.randn(2 * f, d, generator=g) / d ** 0.5).to(td).cuda()
    w3 = (torch.randn(d, f, generator=g) / f ** 0.5).to(td).cuda()
    dy = torch.randn(m, d, generator=g).to(td).cuda()

    def run(api):
        call = (lambda n: getattr(api, n)) if not isinstance(api, dict) else (lambda n: api[n])
        out = {}
        out["y"], out["hid"], out["inv"] = call("add_rmsnorm_forward")(x, res, wn, 1e-6)
        out["dh"], out["dwn"], out["dwn32"] = call("add_rmsnorm_backward")(dy, res, out["hid"], wn, out["inv"], True)
        out["h"], out["gv"] = call("swiglu_fused_forward_save")(x, w12, f)
        out["h2"] = call("swiglu_fused_forward")(x, w12, f)
        out["act"] = call("swiglu_act_forward")(out["gv"], f)
        out["o"] = call("linear_tn")(out["h"], w3)
        out["dw3"] = call("gemm")(dy, out["h"], True, True)
        out["dgv"] = call("swiglu_dh_dgv")(dy, w3, out["gv"], f)
        out["dhid"] = call("gemm")(dy, w3, False, True)
        out["dgv2"] = call("swiglu_fused_backward")(out["dhid"], x, w12, f)
        out["dact"] = call("swiglu_act_backward")(out["dhid"], out["gv"], f)
        out["dx"] = call("gemm")(out["dgv"], w12, False, True)
        buf = torch.empty(m, 2 * f, dtype=td, device="cuda")
        out["dgv_out"] = call("swiglu_dh_dgv")(dy, w3, out["gv"], f, out=buf) if isinstance(api, dict) else call("swiglu_dh_dgv")(dy, w3, out["gv"], f, buf)
        torch.cuda.synchronize()
        return out

    a, b = run(ext), run(py)
    for k in a:
        assert same(a[k], b[k]), f"{k}: the compiled binding and the ctypes route disagree"
    assert ext.device_status(True) == 0


def test_modules_run_on_the_compiled_binding(routes):
    """The public modules pick the extension up when it is built (BINDING == 'pybind')."""
    import mgrrmsnorm_b200.rmsnorm_cuda_ops as ops
    from mgrrmsnorm_b200 import RMSNorm

    assert ops.BINDING == "pybind"
    norm = RMSNorm(1024, epsilon=1e-6).cuda().to(torch.bfloat16)
    x = torch.randn(8, 16, 1024, device="cuda").to(torch.bfloat16).requires_grad_(True)
    norm(x).sum().backward()
    torch.cuda.synchronize()
    assert x.grad is not None and norm.weight.grad is not None


def test_host_cost_per_call(routes, capsys):
    """Host time of one forward + one backward call on a tiny problem (the kernels take ~5 us; the rest is
    the binding). Printed for the record; the only claim checked is that the compiled route is not slower."""
    ext, py = routes
    x = torch.randn(64, 1024, device="cuda").to(torch.bfloat16)
    w = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    dy = torch.randn_like(x)

    def host_us(fwd, bwd, n=2000):
        y, inv = fwd(x, w, 1e-6)
        for _ in range(50):
            fwd(x, w, 1e-6)
            bwd(dy, x, w, inv)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(n):
            fwd(x, w, 1e-6)
            bwd(dy, x, w, inv)
        t1 = time.perf_counter()
        torch.cuda.synchronize()
        return (t1 - t0) / n * 1e6

    best = {"pybind": min(host_us(ext.rmsnorm_forward, ext.rmsnorm_backward) for _ in range(3)),
            "ctypes": min(host_us(py["rmsnorm_forward"], py["rmsnorm_backward"]) for _ in range(3))}
    with capsys.disabled():
        print(f"\n[host cost per forward+backward call pair] pybind {best['pybind']:.1f} us, ctypes {best['ctypes']:.1f} us")
    assert best["pybind"] <= best["ctypes"] * 1.10
