"""RMSNorm folded into the SwiGLU projection (inference form of the pre-norm block): the row-scale kernel, the
scaled epilogue, and PreNormSwiGLU against the two-module path and the fp64 oracle."""
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


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("rows,cols", [(1, 8), (5, 1000), (129, 128), (300, 2048), (2100, 4096), (700, 8192), (40, 16384), (9, 40000)])
def test_row_scales_equal_the_forward_kernels_inv_rms(ops, built_lib, dtype, rows, cols):
    """mgr_rms_inv runs the forward kernels without their output stores: bit-identical inv_rms (except where the
    forward itself takes the bulk-copy ring family, a different summation order, held to the fp32 tolerance)."""
    g = torch.Generator().manual_seed(rows + cols)
    x = torch.randn(rows, cols, generator=g).to(TORCH_DTYPES[dtype]).cuda()
    w = torch.ones(cols, dtype=x.dtype, device="cuda")
    inv = ops.rms_inv(x, 1e-6)
    _, inv_fwd = ops.rmsnorm_forward(x, w, 1e-6)
    torch.cuda.synchronize()
    _, truth = oracle.rmsnorm_fwd(to_np(x), to_np(w), 1e-6)
    assert inv.dtype == torch.float32 and tuple(inv.shape) == (rows,)
    assert np.allclose(to_np(inv), truth, rtol=1e-5, atol=0)
    assert torch.equal(inv, inv_fwd) or np.allclose(to_np(inv), to_np(inv_fwd), rtol=2e-6, atol=0)
    assert built_lib.mgr_device_status(1) == 0


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("m,d,f", [(8, 64, 128), (130, 256, 320), (520, 1024, 1536), (16, 4096, 6912)])
def test_scaled_projection_epilogue(ops, built_lib, dtype, m, d, f):
    """row_scale of ones gives the unscaled kernel's bits; a real scale matches the fp64 formula
    silu(s (x wg^T)) * (s (x wv^T)) within the GEMM tolerance."""
    from tests.test_swiglu_mlp_gpu import gemm_tolerance

    g = torch.Generator().manual_seed(m + d + f)
    td = TORCH_DTYPES[dtype]
    x = torch.randn(m, d, generator=g).to(td).cuda()
    w12 = (torch.randn(2 * f, d, generator=g) / d ** 0.5).to(td).cuda()
    plain = ops.swiglu_fused_forward(x, w12, f)
    ones = ops.swiglu_fused_forward(x, w12, f, row_scale=torch.ones(m, device="cuda"))
    assert torch.equal(plain, ones)
    s = (0.5 + torch.rand(m, generator=g)).cuda()
    got = ops.swiglu_fused_forward(x, w12, f, row_scale=s)
    torch.cuda.synchronize()
    gv = oracle.linear(to_np(x), to_np(w12)) * to_np(s).astype(np.float64)[:, None]
    want = oracle.swiglu_act_fwd(gv, f)
    err = np.abs(to_np(got).astype(np.float64) - want)
    assert float(err.max()) <= gemm_tolerance(d, dtype, float(np.abs(want).max())) + 1e-5, float(err.max())
    with pytest.raises(RuntimeError, match="row_scale"):
        ops.swiglu_fused_forward(x, w12, f, row_scale=torch.ones(m + 1, device="cuda"))
    assert built_lib.mgr_device_status(1) == 0


@pytest.mark.parametrize("dtype", ["f16", "bf16"])
@pytest.mark.parametrize("tokens,d_model", [(96, 256), (16, 1024), (1000, 512)])
def test_prenorm_block_inference_matches_two_modules_and_oracle(built_lib, dtype, tokens, d_model):
    from mgrrmsnorm_b200 import MegaGemmTriton, PreNormSwiGLU, RMSNorm

    td = TORCH_DTYPES[dtype]
    torch.manual_seed(tokens + d_model)
    norm = RMSNorm(d_model, epsilon=1e-6).cuda().to(td)
    mlp = MegaGemmTriton(d_model, multiple_of=128).cuda().to(td)
    g = torch.Generator(device="cuda").manual_seed(5)
    with torch.no_grad():
        norm.weight.copy_((1 + 0.1 * torch.randn(d_model, device="cuda", generator=g)).to(td))
    block = PreNormSwiGLU(norm, mlp)
    x = torch.randn(4, tokens // 4, d_model, device="cuda", generator=g).to(td)
    with torch.no_grad():
        fused = block(x)
        two_step = mlp(norm(x))
    torch.cuda.synchronize()
    assert fused.shape == two_step.shape == x.shape
    # fp64 truth of the block on the same (rounded) parameters
    xf, wf = to_np(x.reshape(-1, d_model)), to_np(norm.weight)
    yn, _ = oracle.rmsnorm_fwd(xf, wf, 1e-6)
    truth = oracle.swiglu_mlp(yn, to_np(mlp.w12.weight), to_np(mlp.w3.weight))["y"]
    scale = max(1.0, float(np.abs(truth).max()))
    for name, got in (("fused", fused), ("two-step", two_step)):
        err = float(np.abs(to_np(got.reshape(-1, d_model)).astype(np.float64) - truth).max())
        assert err < 1e-2 * scale, f"{name}: max err {err:.3e}"
    # with gradients enabled the block is the two modules: same bits as calling them, and differentiable
    xg = x.clone().requires_grad_(True)
    y = block(xg)
    assert torch.equal(y.detach(), two_step)
    y.sum().backward()
    assert xg.grad is not None and norm.weight.grad is not None and mlp.w12.weight.grad is not None
    # the folded weight follows the parameters
    before = block.folded_w12().clone()
    with torch.no_grad():
        norm.weight.mul_(2.0)
        assert not torch.equal(block.folded_w12(), before)
        fused2 = block(x)
        two_step2 = mlp(norm(x))
    assert float((fused2.float() - two_step2.float()).abs().max()) < 1e-2 * max(1.0, float(two_step2.float().abs().max()))
    assert built_lib.mgr_device_status(1) == 0
