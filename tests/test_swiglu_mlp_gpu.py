"""SwiGLU MLP on the tensor-core kernels: the tcgen05 GEMM against exact references on structured
inputs and against the fp64 oracle on random ones; the whole module against the oracle and the golden
vectors of the reference module."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import TORCH_DTYPES, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_lib):
    import rmsnorm_cuda_ops

    return rmsnorm_cuda_ops


def gemm_tolerance(k: int, dtype: str, scale: float) -> float:
    """fp32 accumulation of K products of 16-bit inputs, one rounding to the 16-bit output."""
    half_ulp = 2.0 ** (-11 if dtype == "f16" else -8)
    return scale * (half_ulp + 4e-7 * k ** 0.5) + 1e-6


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 256, 256), (256, 512, 128), (100, 40, 72), (384, 264, 4096),
                                    (1, 8, 8), (300, 1000, 520)])
def test_gemm_integer_inputs_are_exact(ops, built_lib, dtype, m, n, k):
    """Small-integer operands: every product and partial sum is exactly representable, so any tile,
    swizzle or descriptor error shows up as a wrong integer, and the right answer has zero error."""
    g = torch.Generator().manual_seed(m + n + k)
    td = TORCH_DTYPES[dtype]
    a = torch.randint(-2, 3, (m, k), generator=g).to(td)
    b = torch.randint(-2, 3, (n, k), generator=g).to(td)
    c = ops.linear_tn(a.cuda(), b.cuda())
    torch.cuda.synchronize()
    # the fp32 accumulator holds the integer sums exactly; the only rounding is the store to 16 bits
    want = (a.double() @ b.double().t()).to(td)
    assert torch.equal(c.cpu(), want)
    assert built_lib.mgr_device_status(1) == 0


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_gemm_identity_and_one_hot(ops, dtype):
    """B = identity copies A; a one-hot B row picks one column of A: exact, and position-revealing."""
    td = TORCH_DTYPES[dtype]
    g = torch.Generator().manual_seed(3)
    a = torch.randn(200, 512, generator=g).to(td)
    eye = torch.eye(512).to(td)
    assert torch.equal(ops.linear_tn(a.cuda(), eye.cuda()).cpu(), a)
    perm = torch.randperm(512, generator=g)
    assert torch.equal(ops.linear_tn(a.cuda(), eye[perm].cuda()).cpu(), a[:, perm])


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,n,k", [(256, 512, 1024), (520, 264, 4096), (4096, 512, 6912)])
def test_gemm_random_matches_oracle(ops, dtype, m, n, k):
    g = torch.Generator().manual_seed(k)
    td = TORCH_DTYPES[dtype]
    a = torch.randn(m, k, generator=g).to(td)
    b = (torch.randn(n, k, generator=g) / k ** 0.5).to(td)
    c = to_np(ops.linear_tn(a.cuda(), b.cuda())).astype(np.float64)
    want = oracle.linear(to_np(a), to_np(b))
    err = np.abs(c - want)
    assert float(err.max()) <= gemm_tolerance(k, dtype, float(np.abs(want).max())), float(err.max())


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,d,f", [(128, 64, 128), (200, 256, 384), (64, 72, 40), (1024, 4096, 6912), (300, 512, 1000)])
def test_fused_projection_matches_oracle(ops, built_lib, dtype, m, d, f):
    """h = silu(x Wg^T) * (x Wv^T): the fused epilogue against the fp64 formulas (megagemm/swiglu.py:35-41)."""
    g = torch.Generator().manual_seed(m + d + f)
    td = TORCH_DTYPES[dtype]
    x = torch.randn(m, d, generator=g).to(td)
    w12 = (torch.randn(2 * f, d, generator=g) / d ** 0.5).to(td)
    h = to_np(ops.swiglu_fused_forward(x.cuda(), w12.cuda(), f)).astype(np.float64)
    gv = oracle.linear(to_np(x), to_np(w12))
    want = oracle.swiglu_act_fwd(gv, f)
    err = np.abs(h - want)
    assert float(err.max()) <= gemm_tolerance(d, dtype, float(np.abs(want).max())) + 1e-5, float(err.max())
    assert built_lib.mgr_device_status(1) == 0


def test_fused_projection_gate_value_layout(ops):
    """Gate rows are w12[:F], value rows w12[F:] (benchmark_swiglu.py:85-89). With value weights that
    make val == 1 the output is silu(gate); swapping the halves must change it."""
    f, d, m = 256, 128, 128
    x = torch.zeros(m, d)
    x[:, 0] = 1.0
    x[:, 1] = torch.linspace(-4, 4, m)
    w12 = torch.zeros(2 * f, d)
    w12[:f, 1] = 1.0        # gate = x[:, 1]
    w12[f:, 0] = 1.0        # value = 1
    h = ops.swiglu_fused_forward(x.half().cuda(), w12.half().cuda(), f).float().cpu()
    gate = x[:, 1].half().float()
    want = (gate * torch.sigmoid(gate)).half().float()
    assert torch.allclose(h, want[:, None].expand(m, f), atol=2e-3, rtol=2e-3)


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_module_forward_backward_matches_oracle(dtype):
    from megagemm import MegaGemmTriton

    td = TORCH_DTYPES[dtype]
    torch.manual_seed(7)
    mlp = MegaGemmTriton(512, multiple_of=128).cuda().to(td)      # hidden 896
    g = torch.Generator().manual_seed(8)
    x = torch.randn(4, 96, 512, generator=g).to(td)
    dy = torch.randn(4, 96, 512, generator=g).to(td)
    xin = x.cuda().requires_grad_(True)
    y = mlp(xin)
    y.backward(dy.cuda())
    torch.cuda.synchronize()
    out = oracle.swiglu_mlp(to_np(x).reshape(-1, 512), to_np(mlp.w12.weight), to_np(mlp.w3.weight), dy=to_np(dy).reshape(-1, 512))
    # fp16/bf16 MLP against the fp64 truth: 1e-2 max-abs (the bound the reference's own check uses,
    # benchmark_swiglu.py:121-129); weight gradients sum 384 rows and are held to their own scale
    for got, key in ((y.view(-1, 512), "y"), (xin.grad.view(-1, 512), "dx")):
        assert float(np.abs(to_np(got) - out[key]).max()) < 1e-2, key
    for got, key in ((mlp.w12.weight.grad, "dw12"), (mlp.w3.weight.grad, "dw3")):
        err = float(np.abs(to_np(got) - out[key]).max())
        assert err < 1e-2 * max(1.0, float(np.abs(out[key]).max())), (key, err)


def test_module_matches_reference_module_vectors(golden_dir):
    """The fp32 fixture of the reference's MegaGemmTriton (d_model 64, hidden 128), run here in fp16:
    within the reference benchmark's own 1e-2 check of the fp32 outputs."""
    from megagemm import MegaGemmTriton

    g = np.load(golden_dir / "swiglu.npz")
    mlp = MegaGemmTriton(64, multiple_of=32)
    mlp.load_state_dict({"w12.weight": torch.from_numpy(g["mlp_w12"]), "w3.weight": torch.from_numpy(g["mlp_w3"])})
    mlp = mlp.cuda().half()
    x = torch.from_numpy(g["mlp_x"]).half().cuda().requires_grad_(True)
    y = mlp(x)
    y.backward(torch.from_numpy(g["mlp_dy"]).half().cuda())
    assert float((y.float().cpu() - torch.from_numpy(g["mlp_y"])).abs().max()) < 1e-2
    assert float((x.grad.float().cpu() - torch.from_numpy(g["mlp_dx"])).abs().max()) < 1e-2
    assert float((mlp.w12.weight.grad.float().cpu() - torch.from_numpy(g["mlp_dw12"])).abs().max()) < 2e-2
    assert float((mlp.w3.weight.grad.float().cpu() - torch.from_numpy(g["mlp_dw3"])).abs().max()) < 2e-2


def test_fp32_module_keeps_the_reference_structure():
    from megagemm import MegaGemmTriton

    torch.manual_seed(1)
    mlp = MegaGemmTriton(64, multiple_of=32).cuda()
    x = torch.randn(10, 64, device="cuda", requires_grad=True)
    y = mlp(x)
    y.sum().backward()
    out = oracle.swiglu_mlp(to_np(x), to_np(mlp.w12.weight), to_np(mlp.w3.weight))
    assert float(np.abs(to_np(y) - out["y"]).max()) < 1e-3    # TF32-capable library GEMMs in fp32 mode


def test_gemm_argument_errors(built_lib):
    from mgrrmsnorm_b200 import _capi

    P = 0x10000
    assert built_lib.mgr_gemm_tn(P, P, P, 8, 8, 8, 8, 8, 8, _capi.MGR_F32, None) == _capi.MGR_ERR_BAD_DTYPE
    assert built_lib.mgr_gemm_tn(P, P, P, 8, 7, 8, 8, 8, 8, _capi.MGR_F16, None) == _capi.MGR_ERR_BAD_SHAPE
    assert built_lib.mgr_gemm_tn(P, P, P, 8, 8, 8, 4, 8, 8, _capi.MGR_F16, None) == _capi.MGR_ERR_BAD_SHAPE
    assert built_lib.mgr_gemm_tn(None, P, P, 8, 8, 8, 8, 8, 8, _capi.MGR_F16, None) == _capi.MGR_ERR_NULL_PTR
    assert built_lib.mgr_gemm_tn(P + 2, P, P, 8, 8, 8, 8, 8, 8, _capi.MGR_F16, None) == _capi.MGR_ERR_MISALIGNED
    assert built_lib.mgr_swiglu_fused_fwd(P, P, P, 8, 12, 8, _capi.MGR_BF16, None) == _capi.MGR_ERR_BAD_SHAPE
    assert built_lib.mgr_swiglu_fused_fwd(P, P, P, 0, 8, 8, _capi.MGR_BF16, None) == _capi.MGR_OK


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, False), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 192), (200, 264, 328), (72, 40, 4096), (1000, 520, 264)])
def test_gemm_mn_major_operands_integer_exact(ops, built_lib, dtype, a_mn, b_mn, m, n, k):
    """Operands stored transposed ([K, M] / [K, N]) are read in place through MN-major descriptors; with
    small-integer values the product must be exact."""
    g = torch.Generator().manual_seed(m * 3 + n * 5 + k)
    td = TORCH_DTYPES[dtype]
    a = torch.randint(-2, 3, (m, k), generator=g).to(td)
    b = torch.randint(-2, 3, (n, k), generator=g).to(td)
    a_st = a.t().contiguous() if a_mn else a
    b_st = b.t().contiguous() if b_mn else b
    c = ops.gemm(a_st.cuda(), b_st.cuda(), a_mn, b_mn)
    torch.cuda.synchronize()
    assert torch.equal(c.cpu(), (a.double() @ b.double().t()).to(td))
    assert built_lib.mgr_device_status(1) == 0


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,d,f", [(128, 64, 128), (200, 256, 384), (1024, 4096, 6912), (296, 512, 1000)])
def test_fused_backward_matches_oracle(ops, built_lib, dtype, m, d, f):
    """[d_gate | d_val] from dh with the projection recomputed in TMEM, against the fp64 formulas
    (megagemm/swiglu.py:64-76) applied to the fp64 projection."""
    g = torch.Generator().manual_seed(m + d + f + 1)
    td = TORCH_DTYPES[dtype]
    x = torch.randn(m, d, generator=g).to(td)
    w12 = (torch.randn(2 * f, d, generator=g) / d ** 0.5).to(td)
    dh = torch.randn(m, f, generator=g).to(td)
    dgv = to_np(ops.swiglu_fused_backward(dh.cuda(), x.cuda(), w12.cuda(), f)).astype(np.float64)
    gv = oracle.linear(to_np(x), to_np(w12))
    want = oracle.swiglu_act_bwd(to_np(dh), gv, f)
    err = np.abs(dgv - want)
    assert float(err.max()) <= gemm_tolerance(d, dtype, float(np.abs(want).max())) + 1e-4, float(err.max())
    assert built_lib.mgr_device_status(1) == 0


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_config4_shape_forward_backward(dtype):
    """d_model 4096, hidden 6912 (the module's default for that d_model), 1024 of the 4096 tokens: the
    module on the tensor-core kernels against the same formulas evaluated by library GEMMs in fp32."""
    from megagemm import MegaGemmTriton

    td = TORCH_DTYPES[dtype]
    torch.manual_seed(1234)
    mlp = MegaGemmTriton(4096).cuda().to(td)
    assert mlp.hidden == 6912
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(8, 128, 4096, device="cuda", generator=g).to(td)
    dy = torch.randn(8, 128, 4096, device="cuda", generator=g).to(td)
    xin = x.clone().requires_grad_(True)
    y = mlp(xin)
    y.backward(dy)
    w12, w3 = mlp.w12.weight.detach().float(), mlp.w3.weight.detach().float()
    xr = x.float().requires_grad_(True)
    w12r, w3r = w12.clone().requires_grad_(True), w3.clone().requires_grad_(True)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        gv = torch.nn.functional.linear(xr, w12r)
        yr = torch.nn.functional.linear(torch.nn.functional.silu(gv[..., :6912]) * gv[..., 6912:], w3r)
        yr.backward(dy.float())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    assert float((y.float() - yr).abs().max()) < 1e-2
    assert float((xin.grad.float() - xr.grad).abs().max()) < 1e-2
    for got, want in ((mlp.w12.weight.grad, w12r.grad), (mlp.w3.weight.grad, w3r.grad)):
        scale = max(1.0, float(want.abs().max()))
        assert float((got.float() - want).abs().max()) < 1e-2 * scale


def _fp32_library_mlp(x, w12, w3, dy, f):
    """The reference's formulas (w12 -> silu(gate) * value -> w3, megagemm/swiglu.py:35-41,166-169) evaluated by
    library GEMMs in fp32 (no tf32) on the GPU, with autograd for the backward: the truth proxy for problems too
    large for the fp64 CPU oracle. Returns y, dx, dw12, dw3 in fp32."""
    xr = x.float().requires_grad_(True)
    w12r, w3r = w12.float().requires_grad_(True), w3.float().requires_grad_(True)
    prev = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        gv = torch.nn.functional.linear(xr, w12r)
        yr = torch.nn.functional.linear(torch.nn.functional.silu(gv[..., :f]) * gv[..., f:], w3r)
        yr.backward(dy.float())
    finally:
        torch.backends.cuda.matmul.allow_tf32 = prev
    return yr.detach(), xr.grad, w12r.grad, w3r.grad


def _check_mlp_against_library_and_oracle(mlp, x, dy, dtype, sample_rows):
    """Whole tensors against the fp32 library evaluation; `sample_rows` rows of y and dx (rows of an MLP are
    independent given the weights) against the fp64 CPU oracle, which also anchors the library proxy."""
    f = mlp.hidden
    xin = x.clone().requires_grad_(True)
    y = mlp(xin)
    y.backward(dy)
    torch.cuda.synchronize()
    w12, w3 = mlp.w12.weight.detach(), mlp.w3.weight.detach()
    yr, dxr, dw12r, dw3r = _fp32_library_mlp(x, w12, w3, dy, f)
    m, d = x.shape
    # activations: one output rounding + fp32 accumulation over the contraction lengths involved
    for name, got, want, k in (("y", y, yr, f), ("dx", xin.grad, dxr, 2 * f)):
        tol = gemm_tolerance(k, dtype, float(want.abs().max())) * 2 + 1e-4      # x2: the 16-bit intermediates h / dgv
        err = float((got.float() - want).abs().max())
        assert err <= max(tol, 1e-2 if float(want.abs().max()) < 4 else tol), f"{name}: max err {err:.3e} > {tol:.3e}"
        assert err < 1e-2 * max(1.0, float(want.abs().max())), name
    # weight gradients contract over the m tokens
    for name, got, want in (("dw12", mlp.w12.weight.grad, dw12r), ("dw3", mlp.w3.weight.grad, dw3r)):
        tol = gemm_tolerance(m, dtype, float(want.abs().max())) * 2 + 1e-4
        err = float((got.float() - want).abs().max())
        assert err <= tol, f"{name}: max err {err:.3e} > {tol:.3e} (max |truth| {float(want.abs().max()):.3g})"
    # fp64 oracle on sampled rows (first tile, a tile edge, the last rows)
    rows = torch.tensor(sample_rows, device=x.device)
    o = oracle.swiglu_mlp(to_np(x[rows]), to_np(w12), to_np(w3), dy=to_np(dy[rows]))
    for name, got, want, k in (("y", y[rows], o["y"], f), ("dx", xin.grad[rows], o["dx"], 2 * f)):
        err = float(np.abs(to_np(got).astype(np.float64) - want).max())
        tol = gemm_tolerance(k, dtype, float(np.abs(want).max())) * 2 + 1e-4
        assert err <= tol, f"{name} vs fp64 oracle on sampled rows: {err:.3e} > {tol:.3e}"
        lib = float(np.abs(to_np((yr if name == "y" else dxr)[rows]).astype(np.float64) - want).max())
        assert lib <= 1e-4 * max(1.0, float(np.abs(want).max())), f"the fp32 library proxy is off the oracle by {lib:.3e}"


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
def test_config4_full_size(built_lib, dtype):
    """Config 4 at its full size: x [32,128,4096] (4096 tokens), d_model 4096, hidden 6912 (the module's default),
    nn.Linear default init from a seed, forward + backward through the module."""
    from megagemm import MegaGemmTriton

    td = TORCH_DTYPES[dtype]
    torch.manual_seed(1234)
    mlp = MegaGemmTriton(4096).cuda().to(td)
    assert mlp.hidden == 6912
    g = torch.Generator(device="cuda").manual_seed(1234)
    x = torch.randn(4096, 4096, device="cuda", generator=g).to(td)
    dy = torch.randn(4096, 4096, device="cuda", generator=g).to(td)
    _check_mlp_against_library_and_oracle(mlp, x, dy, dtype, [0, 1, 127, 128, 255, 256, 2047, 2048, 4094, 4095])
    assert built_lib.mgr_device_status(1) == 0


def test_config5_rank_slice_full_size(built_lib):
    """One rank's share of config 5 at 8 GPUs: bf16, 16384 tokens, d_model 8192, 3584 of the 28672 hidden units
    (w12 slice [7168, 8192], w3 slice [8192, 3584]); all six GEMMs at their real sizes, including the two weight
    gradients that contract over 16384 tokens and the 128 / 64 row-tile walks of the projection."""
    from mgrrmsnorm_b200 import sharding

    td = torch.bfloat16
    d, f_full, world, m = 8192, 28672, 8, 16384
    tp = sharding.TensorParallelSwiGLU(d, f_full, world, rank=3).cuda().to(td)
    mlp = tp.local
    f = mlp.hidden
    assert f == 3584
    g = torch.Generator(device="cuda").manual_seed(99)
    with torch.no_grad():       # nn.Linear default init; fan_in of w3 is the FULL d_ff
        mlp.w12.weight.copy_((torch.rand(2 * f, d, device="cuda", generator=g) * 2 - 1) / d ** 0.5)
        mlp.w3.weight.copy_((torch.rand(d, f, device="cuda", generator=g) * 2 - 1) / f_full ** 0.5)
    x = torch.randn(m, d, device="cuda", generator=g).to(td)
    dy = torch.randn(m, d, device="cuda", generator=g).to(td)
    _check_mlp_against_library_and_oracle(mlp, x, dy, "bf16", [0, 127, 128, 8191, 8192, 16383])
    assert built_lib.mgr_device_status(1) == 0


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,d,f", [(128, 64, 128), (200, 256, 384), (1024, 4096, 6912), (296, 512, 1000)])
def test_kept_projection_forward_and_fused_dh_backward(ops, built_lib, dtype, m, d, f):
    """Training pair: the forward that also stores [gate | val], and the dh = dy w3 GEMM whose epilogue
    turns dh (fp32, in tensor memory) and the stored projection into [d_gate | d_val]."""
    g = torch.Generator().manual_seed(m + d + f + 2)
    td = TORCH_DTYPES[dtype]
    x = torch.randn(m, d, generator=g).to(td)
    w12 = (torch.randn(2 * f, d, generator=g) / d ** 0.5).to(td)
    w3 = (torch.randn(d, f, generator=g) / f ** 0.5).to(td)
    dy = torch.randn(m, d, generator=g).to(td)
    h, gv = ops.swiglu_fused_forward_save(x.cuda(), w12.cuda(), f)
    assert torch.equal(h, ops.swiglu_fused_forward(x.cuda(), w12.cuda(), f)), "h must not depend on whether gv is kept"
    gv64 = oracle.linear(to_np(x), to_np(w12))
    err = np.abs(to_np(gv).astype(np.float64) - gv64)
    assert float(err.max()) <= gemm_tolerance(d, dtype, float(np.abs(gv64).max())), float(err.max())
    # backward from the STORED (rounded) projection, like the reference's kernel reads w12_out
    dgv = to_np(ops.swiglu_dh_dgv(dy.cuda(), w3.cuda(), gv, f)).astype(np.float64)
    dh64 = to_np(dy).astype(np.float64) @ to_np(w3).astype(np.float64)
    want = oracle._act_bwd_f64(dh64, to_np(gv).astype(np.float64), f)
    err = np.abs(dgv - want)
    assert float(err.max()) <= gemm_tolerance(d, dtype, float(np.abs(want).max())) + 1e-4, float(err.max())
    assert built_lib.mgr_device_status(1) == 0


@pytest.mark.parametrize("recompute", ["0", "1"])
def test_module_backward_modes_agree_with_oracle(monkeypatch, recompute):
    """MGR_MLP_RECOMPUTE selects between keeping the projection and recomputing it; both must meet the
    same tolerances against the fp64 oracle."""
    from megagemm import MegaGemmTriton

    monkeypatch.setenv("MGR_MLP_RECOMPUTE", recompute)
    torch.manual_seed(11)
    mlp = MegaGemmTriton(256, multiple_of=128).cuda().bfloat16()
    g = torch.Generator().manual_seed(12)
    x = torch.randn(3, 64, 256, generator=g).bfloat16()
    dy = torch.randn(3, 64, 256, generator=g).bfloat16()
    xin = x.cuda().requires_grad_(True)
    y = mlp(xin)
    y.backward(dy.cuda())
    out = oracle.swiglu_mlp(to_np(x).reshape(-1, 256), to_np(mlp.w12.weight), to_np(mlp.w3.weight), dy=to_np(dy).reshape(-1, 256))
    assert float(np.abs(to_np(y).reshape(-1, 256) - out["y"]).max()) < 2e-2
    assert float(np.abs(to_np(xin.grad).reshape(-1, 256) - out["dx"]).max()) < 2e-2
    for got, key in ((mlp.w12.weight.grad, "dw12"), (mlp.w3.weight.grad, "dw3")):
        assert float(np.abs(to_np(got) - out[key]).max()) < 2e-2 * max(1.0, float(np.abs(out[key]).max())), key
    with torch.no_grad():
        assert torch.equal(mlp(x.cuda()), y.detach()), "inference forward must equal the training forward"


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,d,f", [(256, 64, 128), (128, 128, 256), (520, 256, 384), (1024, 1024, 1536), (296, 512, 1000)])
def test_cta_pair_kernels_equal_single_cta_kernels(ops, built_lib, mgr_env, dtype, m, d, f):
    """MGR_GEMM_CTA_GROUP=2 runs every GEMM on pairs of CTAs sharing one MMA (256-row tiles, each CTA
    loading half of B). The K order of the accumulation is the same, so every output must be bit-identical
    to the single-CTA kernels' -- for all operand layouts and all epilogues."""
    g = torch.Generator().manual_seed(m + d + f + 3)
    td = TORCH_DTYPES[dtype]
    x = torch.randn(m, d, generator=g).to(td).cuda()
    w12 = (torch.randn(2 * f, d, generator=g) / d ** 0.5).to(td).cuda()
    w3 = (torch.randn(d, f, generator=g) / f ** 0.5).to(td).cuda()
    dy = torch.randn(m, d, generator=g).to(td).cuda()

    def everything():
        h, gv = ops.swiglu_fused_forward_save(x, w12, f)
        out = {"h": h, "gv": gv, "h2": ops.swiglu_fused_forward(x, w12, f), "y": ops.linear_tn(h, w3)}
        out["dh"] = ops.gemm(dy, w3, False, True)
        out["dw3"] = ops.gemm(dy, h, True, True)
        out["dgv"] = ops.swiglu_dh_dgv(dy, w3, gv, f)
        out["dgv2"] = ops.swiglu_fused_backward(out["dh"], x, w12, f)
        out["dx"] = ops.gemm(out["dgv"], w12, False, True)
        out["dw12"] = ops.gemm(out["dgv"], x, True, True)
        out["mn_k"] = ops.gemm(x.t().contiguous(), w12, True, False)     # MN-major A with K-major B
        torch.cuda.synchronize()
        return out

    mgr_env("MGR_GEMM_CTA_GROUP", "1")
    one = everything()
    mgr_env("MGR_GEMM_CTA_GROUP", "2")
    two = everything()
    assert built_lib.mgr_device_status(1) == 0
    for k in one:
        assert torch.equal(one[k], two[k]), f"{k}: pair kernel differs, max |diff| {float((one[k].float() - two[k].float()).abs().max())}"


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,d,f", [(8, 64, 128), (16, 512, 1000), (64, 4096, 6912), (130, 256, 320), (600, 1024, 1536),
                                   # short A boxes whose contraction wraps the (run-time sized) stage ring several times
                                   (8, 4096, 1024), (1, 2048, 256), (24, 2048, 512), (56, 1600, 384), (120, 1536, 256)])
def test_narrow_tile_kernels_equal_wide_tile_kernels(ops, built_lib, mgr_env, dtype, m, d, f):
    """Skinny problems run on 96-, 64- or 32-column tiles (MGR_GEMM_NARROW=96 / =1 / =32 forces them, =0 forbids
    them; 96 = 48 gate + 48 value columns exists for the fused projection only, the plain GEMM then takes 64) so
    that more CTAs share the weight stream. Same K order, so the fused projection and the plain GEMM must be
    bit-identical to the 256-column kernels."""
    g = torch.Generator().manual_seed(m + d + f + 4)
    td = TORCH_DTYPES[dtype]
    x = torch.randn(m, d, generator=g).to(td).cuda()
    w12 = (torch.randn(2 * f, d, generator=g) / d ** 0.5).to(td).cuda()
    w3 = (torch.randn(d, f, generator=g) / f ** 0.5).to(td).cuda()
    outs = {}
    for narrow in ("0", "1", "32", "96"):
        mgr_env("MGR_GEMM_NARROW", narrow)
        mgr_env("MGR_GEMM_CTA_GROUP", "1")
        h = ops.swiglu_fused_forward(x, w12, f)
        outs[narrow] = (h, ops.linear_tn(h, w3))
        torch.cuda.synchronize()
    assert built_lib.mgr_device_status(1) == 0
    for narrow in ("1", "32", "96"):
        assert torch.equal(outs["0"][0], outs[narrow][0]), f"fused projection differs with tile width {narrow}"
        assert torch.equal(outs["0"][1], outs[narrow][1]), f"plain GEMM differs with tile width {narrow}"
    gv = oracle.linear(to_np(x), to_np(w12))
    want = oracle.swiglu_act_fwd(gv, f)
    err = np.abs(to_np(outs["1"][0]).astype(np.float64) - want)
    assert float(err.max()) <= gemm_tolerance(d, dtype, float(np.abs(want).max())) + 1e-5
