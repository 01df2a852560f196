"""SwiGLU activation parity on the GPU (C ABI via the operator API) against the oracle and the
vectors produced by the reference's Triton kernels."""
import numpy as np
import pytest
import torch

from oracle import oracle
from tests.util import TORCH_DTYPES, assert_matches_truth, to_np

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(built_lib):
    import rmsnorm_cuda_ops

    return rmsnorm_cuda_ops


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("m,f", [(1, 1), (3, 7), (9, 96), (64, 1000), (33, 6912), (512, 2048)])
def test_activation_matches_oracle(ops, dtype, m, f):
    g = torch.Generator().manual_seed(m * 1000 + f)
    td = TORCH_DTYPES[dtype]
    gv = (1.5 * torch.randn(m, 2 * f, generator=g)).to(td)
    dh = torch.randn(m, f, generator=g).to(td)
    h = ops.swiglu_act_forward(gv.cuda(), f)
    dgv = ops.swiglu_act_backward(dh.cuda(), gv.cuda(), f)
    torch.cuda.synchronize()
    assert_matches_truth(h, oracle.swiglu_act_fwd(to_np(gv), f), dtype, "h", slack=2.0)
    assert_matches_truth(dgv, oracle.swiglu_act_bwd(to_np(dh), to_np(gv), f), dtype, "dgv", slack=2.0)


@pytest.mark.parametrize("case,dtype", [("act_f32", "f32"), ("act_f16", "f16"), ("act_bf16", "bf16")])
def test_activation_matches_reference_triton_vectors(ops, golden_dir, case, dtype):
    """Outputs of _mg_swiglu_fwd_kernel / _mg_swiglu_bwd_kernel stored in tests/golden/swiglu.npz. Both
    sides round an fp32 result to the tensor dtype, so they may differ by one output ulp at most."""
    g = np.load(golden_dir / "swiglu.npz")
    td = TORCH_DTYPES[dtype]
    gv = torch.from_numpy(g[f"{case}_gv"]).to(td).cuda()
    dh = torch.from_numpy(g[f"{case}_dh"]).to(td).cuda()
    f = gv.shape[1] // 2
    h = to_np(ops.swiglu_act_forward(gv, f))
    dgv = to_np(ops.swiglu_act_backward(dh, gv, f))
    for got, want, name in ((h, g[f"{case}_h"], "h"), (dgv, g[f"{case}_dgv"], "dgv")):
        if dtype == "f32":
            np.testing.assert_allclose(got, want, rtol=1e-5, atol=1e-6, err_msg=name)
        else:
            assert bool((np.abs(got - want) <= oracle.ulp_of(want, dtype)).all()), name


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_function_autograd_nd(dtype):
    from megagemm import MegaGemmFunction

    td = TORCH_DTYPES[dtype]
    g = torch.Generator().manual_seed(5)
    gv = torch.randn(4, 10, 2 * 64, generator=g).to(td)
    dh = torch.randn(4, 10, 64, generator=g).to(td)
    a = gv.cuda().requires_grad_(True)
    h = MegaGemmFunction.apply(a, 64)
    assert h.shape == (4, 10, 64)
    h.backward(dh.cuda())
    assert_matches_truth(h.view(-1, 64), oracle.swiglu_act_fwd(to_np(gv).reshape(-1, 128), 64), dtype, "h", slack=2.0)
    assert_matches_truth(a.grad.view(-1, 128), oracle.swiglu_act_bwd(to_np(dh).reshape(-1, 64), to_np(gv).reshape(-1, 128), 64),
                         dtype, "dgv", slack=2.0)
