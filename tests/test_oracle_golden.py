"""Pins the CPU oracle against vectors produced by the reference's own code (tests/golden/*.npz,
written by tests/golden/make_golden.py). CPU only."""
import numpy as np
import pytest

from oracle import oracle


@pytest.fixture(scope="module")
def rms(golden_dir):
    return np.load(golden_dir / "rmsnorm.npz")


@pytest.fixture(scope="module")
def swi(golden_dir):
    return np.load(golden_dir / "swiglu.npz")


@pytest.mark.parametrize("case", ["f32_a", "f32_b", "f16", "bf16"])
def test_forward_restatement_is_bit_exact_with_reference_cpu(rms, case):
    """mgr_oracle_rmsnorm_fwd_f32seq vs the reference's rmsnorm_cpu output (rmsnorm_standalone.cu:17-30)."""
    y = oracle.rmsnorm_fwd_f32seq(rms[f"{case}_x"], rms[f"{case}_w"], float(rms[f"{case}_eps"]))
    assert np.array_equal(y, rms[f"{case}_y_refcpu"])


@pytest.mark.parametrize("case", ["f32_a", "f32_b", "f16", "bf16"])
def test_truth_matches_reference_formula(rms, case):
    """fp64 oracle vs the formula the reference's test differentiates (test_rmsnorm.py:55-60), fwd and bwd."""
    x, w, dy, eps = rms[f"{case}_x"], rms[f"{case}_w"], rms[f"{case}_dy"], float(rms[f"{case}_eps"])
    y, _ = oracle.rmsnorm_fwd(x, w, eps)
    dx, dw = oracle.rmsnorm_bwd(dy, x, w, eps)
    np.testing.assert_allclose(y, rms[f"{case}_y"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(dx, rms[f"{case}_dx"], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(dw, rms[f"{case}_dw"], rtol=1e-10, atol=1e-12)
    # and the reference's fp32 CPU forward sits within fp32 rounding of that truth
    np.testing.assert_allclose(rms[f"{case}_y_refcpu"], y, rtol=2e-6, atol=1e-6)


def test_live_reference_library_agrees_with_fixture(rms):
    """When oracle/_ref is present, its rmsnorm_cpu must reproduce the committed fixture bit for bit."""
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libmgr_ref.so not built (no reference tree on this machine)")
    y = ref.cpu_forward(rms["f32_a_x"], rms["f32_a_w"], float(rms["f32_a_eps"]))
    assert np.array_equal(y, rms["f32_a_y_refcpu"])


def test_live_reference_cpu_forward_is_reproduced_on_random_shapes():
    """The reference's compiled rmsnorm_cpu (rmsnorm_standalone.cu:17-30) against the restatement on seeded
    random shapes, value scales and epsilons: bit-exact every time, and within fp32 rounding of the fp64 truth."""
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref/libmgr_ref.so not built (no reference tree on this machine)")
    rng = np.random.default_rng(2024)
    for _ in range(25):
        rows = int(rng.integers(1, 40))
        cols = int(rng.choice([1, 2, 7, 8, 64, 100, 255, 256, 1000, 1024, 4096, 5120]))
        scale = float(rng.choice([1e-3, 1.0, 30.0]))
        eps = float(rng.choice([1e-5, 1e-6, 1e-12]))
        x = (scale * rng.standard_normal((rows, cols))).astype(np.float32)
        w = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
        want = ref.cpu_forward(x, w, eps)
        got = oracle.rmsnorm_fwd_f32seq(x, w, eps)
        assert np.array_equal(got, want), (rows, cols, scale, eps)
        truth, _ = oracle.rmsnorm_fwd(x, w, eps)
        np.testing.assert_allclose(want, truth, rtol=4e-6, atol=1e-6 * scale)


@pytest.mark.parametrize("case,tol", [("act_f32", 2e-6), ("act_f16", 2e-3), ("act_bf16", 1.6e-2)])
def test_activation_matches_reference_triton_kernels(swi, case, tol):
    """fp64 oracle vs _mg_swiglu_fwd_kernel / _mg_swiglu_bwd_kernel outputs (megagemm/swiglu.py:18-79).
    The reference stores in the tensor dtype, so the half cases differ from the truth by one rounding."""
    gv, dh = swi[f"{case}_gv"], swi[f"{case}_dh"]
    f = gv.shape[1] // 2
    h = oracle.swiglu_act_fwd(gv, f)
    dgv = oracle.swiglu_act_bwd(dh, gv, f)
    np.testing.assert_allclose(swi[f"{case}_h"], h, rtol=tol, atol=tol)
    np.testing.assert_allclose(swi[f"{case}_dgv"], dgv, rtol=tol, atol=tol)


def test_mlp_matches_reference_module(swi):
    """fp64 MLP oracle vs MegaGemmTriton fwd+bwd and vs PyTorchSwiGLU (benchmark_swiglu.py:40-58, 85-89)."""
    out = oracle.swiglu_mlp(swi["mlp_x"].reshape(-1, 64), swi["mlp_w12"], swi["mlp_w3"], dy=swi["mlp_dy"].reshape(-1, 64))
    assert int(swi["mlp_hidden"]) == swi["mlp_w3"].shape[1] == 128
    np.testing.assert_allclose(swi["mlp_y"].reshape(-1, 64), out["y"], rtol=1e-4, atol=2e-6)
    np.testing.assert_allclose(swi["mlp_y_pytorchswiglu"].reshape(-1, 64), out["y"], rtol=1e-4, atol=2e-6)
    np.testing.assert_allclose(swi["mlp_dx"].reshape(-1, 64), out["dx"], rtol=1e-4, atol=2e-6)
    np.testing.assert_allclose(swi["mlp_dw12"], out["dw12"], rtol=1e-4, atol=5e-6)
    np.testing.assert_allclose(swi["mlp_dw3"], out["dw3"], rtol=1e-4, atol=5e-6)


def test_linear_c_restatement(swi):
    a = swi["mlp_x"].reshape(-1, 64)
    b = swi["mlp_w12"]
    c = np.empty((a.shape[0], b.shape[0]), np.float64)
    oracle.lib().mgr_oracle_linear_f64(c.ctypes.data, np.ascontiguousarray(a).ctypes.data,
                                       np.ascontiguousarray(b).ctypes.data, a.shape[0], b.shape[0], a.shape[1])
    np.testing.assert_allclose(c, oracle.linear(a, b), rtol=1e-12, atol=1e-14)


def test_round_to_matches_torch():
    import torch

    rng = np.random.default_rng(0)
    a = (rng.standard_normal(10000) * 10 ** rng.uniform(-6, 4, 10000)).astype(np.float32)
    t = torch.from_numpy(a)
    assert np.array_equal(oracle.round_to(a, "bf16"), t.to(torch.bfloat16).float().numpy())
    assert np.array_equal(oracle.round_to(a, "f16"), t.to(torch.float16).float().numpy())
    assert oracle.ulp_of(np.array([1.0]), "bf16")[0] == 2.0 ** -7
    assert oracle.ulp_of(np.array([5.0]), "f16")[0] == 2.0 ** -8


@pytest.mark.parametrize("case", ["f32", "f16", "bf16"])
def test_add_rmsnorm_composition_matches_reference_sequence(golden_dir, case):
    """Residual add + norm as a user of the reference writes it (torch add, then the reference's CPU forward /
    the formula its test differentiates): the oracle's restatement of that sequence -- round(x + residual)
    in the case's dtype, then the pinned norm oracle; backward = norm backward + the residual-stream
    gradient -- reproduces the fixture."""
    z = np.load(golden_dir / "add_rmsnorm.npz")
    x, res, w, dy, dres = (z[f"{case}_{k}"] for k in ("x", "res", "w", "dy", "dres"))
    eps = float(z[f"{case}_eps"])
    h = oracle.round_to(x + res, case)
    assert np.array_equal(h, z[f"{case}_h"])
    assert np.array_equal(oracle.rmsnorm_fwd_f32seq(h, w, eps), z[f"{case}_y_refcpu"])
    y, _ = oracle.rmsnorm_fwd(h, w, eps)
    dx, dw = oracle.rmsnorm_bwd(dy, h, w, eps)
    np.testing.assert_allclose(y, z[f"{case}_y"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(dx + dres.astype(np.float64), z[f"{case}_dh"], rtol=1e-10, atol=1e-12)
    np.testing.assert_allclose(dw, z[f"{case}_dw"], rtol=1e-10, atol=1e-12)


_LIVE_TRITON_SCRIPT = r"""
import os, sys
os.environ["TRITON_INTERPRET"] = "1"
ref_dir, out_path = sys.argv[1], sys.argv[2]
sys.path.insert(0, ref_dir)
import numpy as np, torch
from megagemm.swiglu import MegaGemmFunction          # the reference package, unmodified
g = torch.Generator().manual_seed(777)
out = {}
for i, (m, f, dt) in enumerate([(3, 32, torch.float32), (7, 96, torch.float32), (5, 160, torch.float16),
                                (4, 256, torch.bfloat16), (1, 8, torch.float32), (6, 1000, torch.float16)]):
    gv = (2.0 * torch.randn(m, 2 * f, generator=g)).to(dt).requires_grad_(True)
    dh = torch.randn(m, f, generator=g).to(dt)
    h = MegaGemmFunction.apply(gv, f)
    h.backward(dh)
    out[f"c{i}_f"] = np.int64(f)
    out[f"c{i}_dtype"] = np.array(str(dt).split(".")[1])
    out[f"c{i}_gv"] = gv.detach().float().numpy(); out[f"c{i}_dh"] = dh.float().numpy()
    out[f"c{i}_h"] = h.detach().float().numpy(); out[f"c{i}_dgv"] = gv.grad.float().numpy()
np.savez(out_path, **out)
"""


def test_live_reference_triton_kernels_on_random_inputs(tmp_path):
    """Where the reference tree is present (this never runs on the GPU box): its Triton kernels
    (_mg_swiglu_fwd_kernel / _mg_swiglu_bwd_kernel, megagemm/swiglu.py:18-79) executed by the Triton interpreter
    on fresh random inputs, against the oracle. Outputs are stored in the input dtype; the bound is one unit in
    the last place of that dtype (the interpreter's narrowing conversion is not always round-to-nearest-even)
    plus fp32 evaluation error."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    # the reference tree: MGR_REFERENCE_DIR, else a directory `reference` beside this repository
    ref_dir = Path(os.environ.get("MGR_REFERENCE_DIR") or Path(__file__).resolve().parents[2] / "reference")
    if not (ref_dir / "megagemm" / "swiglu.py").exists():
        pytest.skip("reference tree not present on this machine")
    out_path = tmp_path / "live.npz"
    run = subprocess.run([sys.executable, "-c", _LIVE_TRITON_SCRIPT, str(ref_dir), str(out_path)], capture_output=True,
                         text=True, timeout=600)
    if run.returncode != 0 and "triton" in (run.stderr or "").lower() and "interpret" in (run.stderr or "").lower():
        pytest.skip("Triton interpreter unavailable: " + run.stderr[-200:])
    assert run.returncode == 0, run.stderr[-1500:]
    z = np.load(out_path)
    n = len([k for k in z.files if k.endswith("_f")])
    assert n == 6
    for i in range(n):
        f = int(z[f"c{i}_f"])
        dtype = {"float32": "f32", "float16": "f16", "bfloat16": "bf16"}[str(z[f"c{i}_dtype"])]
        gv, dh = z[f"c{i}_gv"], z[f"c{i}_dh"]
        for got, truth in ((z[f"c{i}_h"], oracle.swiglu_act_fwd(gv, f)), (z[f"c{i}_dgv"], oracle.swiglu_act_bwd(dh, gv, f))):
            bound = oracle.ulp_of(truth, dtype) * (0 if dtype == "f32" else 1) + 4e-6 * np.abs(truth) + 1e-6
            assert (np.abs(got.astype(np.float64) - truth) <= bound).all(), (i, dtype, float(np.abs(got - truth).max()))


def test_oracle_backward_formulas_against_finite_differences():
    """Independent of torch autograd: the oracle's closed-form backward (src/rmsnorm_kernel.cu:258-312 for the
    norm, megagemm/swiglu.py:64-76 for the activation) against central differences of its own forward, in fp64."""
    rng = np.random.default_rng(5)
    rows, cols, eps = 3, 24, 1e-6
    x = rng.standard_normal((rows, cols)).astype(np.float32)
    w = (1 + 0.1 * rng.standard_normal(cols)).astype(np.float32)
    dy = rng.standard_normal((rows, cols)).astype(np.float32)

    def loss(xx, ww):
        xx = xx.astype(np.float64); ww = ww.astype(np.float64)
        inv = 1.0 / np.sqrt((xx * xx).mean(axis=1, keepdims=True) + float(np.float32(eps)))
        return float((xx * inv * ww * dy).sum())

    dx, dw = oracle.rmsnorm_bwd(dy, x, w, eps)
    h = 1e-4
    for (r, c) in [(0, 0), (1, 7), (2, 23)]:
        xp, xm = x.astype(np.float64).copy(), x.astype(np.float64).copy()
        xp[r, c] += h; xm[r, c] -= h
        assert abs((loss(xp, w) - loss(xm, w)) / (2 * h) - dx[r, c]) < 1e-6
    for c in (0, 11, 23):
        wp, wm = w.astype(np.float64).copy(), w.astype(np.float64).copy()
        wp[c] += h; wm[c] -= h
        assert abs((loss(x, wp) - loss(x, wm)) / (2 * h) - dw[c]) < 1e-6

    m, f = 4, 10
    gv = (1.5 * rng.standard_normal((m, 2 * f))).astype(np.float32)
    dh = rng.standard_normal((m, f)).astype(np.float32)

    def act_loss(g):
        g = g.astype(np.float64)
        gate, val = g[:, :f], g[:, f:]
        return float((gate / (1 + np.exp(-gate)) * val * dh).sum())

    dgv = oracle.swiglu_act_bwd(dh, gv, f)
    for (r, c) in [(0, 0), (2, f - 1), (1, f), (3, 2 * f - 1)]:
        gp, gm = gv.astype(np.float64).copy(), gv.astype(np.float64).copy()
        gp[r, c] += h; gm[r, c] -= h
        assert abs((act_loss(gp) - act_loss(gm)) / (2 * h) - dgv[r, c]) < 1e-6
