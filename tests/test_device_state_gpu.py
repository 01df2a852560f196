"""Device-side state of the library as the host sees it: the status word a kernel sets when one of its bounded
waits runs out, and the scratch the allocation-free backward may need. Nothing here makes a kernel wait, trap
or fault: the status word is written from the host through the library's test hook."""
import pytest
import torch

from mgrrmsnorm_b200 import _capi

pytestmark = pytest.mark.gpu


def test_timeout_status_is_reported_until_cleared(built_lib):
    L = built_lib
    assert L.mgr_device_status(1) == _capi.MGR_OK
    for family in (0, 1):                      # RMSNorm ring kernels' word, GEMM kernels' word
        assert L.mgr_debug_poke_device_status(family, _capi.MGR_ERR_DEVICE_TIMEOUT) == _capi.MGR_OK
        assert L.mgr_device_status(0) == _capi.MGR_ERR_DEVICE_TIMEOUT      # a read that does not clear
        assert L.mgr_device_status(0) == _capi.MGR_ERR_DEVICE_TIMEOUT
        assert L.mgr_device_status(1) == _capi.MGR_ERR_DEVICE_TIMEOUT      # reported, then cleared
        assert L.mgr_device_status(1) == _capi.MGR_OK
    assert L.mgr_debug_poke_device_status(2, 0) == _capi.MGR_ERR_BAD_SHAPE


def test_python_layer_raises_on_a_timeout_status(built_lib):
    import rmsnorm_cuda_ops as ops

    ops.device_status()                         # clean: returns
    built_lib.mgr_debug_poke_device_status(1, _capi.MGR_ERR_DEVICE_TIMEOUT)
    with pytest.raises(_capi.MgrStatusError, match="bounded device-side wait"):
        ops.device_status()
    ops.device_status()                         # the raising read cleared it
    # kernels launched after a cleared status run normally
    x = torch.randn(64, 1024, device="cuda").bfloat16()
    y, _ = ops.rmsnorm_forward(x, torch.ones(1024, device="cuda", dtype=torch.bfloat16), 1e-6)
    torch.cuda.synchronize()
    assert torch.isfinite(y.float()).all()
    ops.device_status()


def test_every_row_length_up_to_16384_fits_the_fixed_scratch(built_lib):
    """mgr_rmsnorm_bwd_noalloc refuses problems whose partial rows exceed MGR_NOALLOC_SCRATCH_BYTES (16 MiB). The
    number of partial rows is SMs x resident CTAs of the kernel chosen for the row length, so the bound is a
    property of the device: on this GPU every packet-sized row length up to 16384 columns must fit, for all
    three dtypes, however many rows there are. Host-only queries; nothing is launched."""
    L = built_lib
    limit = 16 << 20
    worst = (0, None)
    for code, name in ((_capi.MGR_F32, "f32"), (_capi.MGR_F16, "f16"), (_capi.MGR_BF16, "bf16")):
        for cols in range(8, 16384 + 1, 8):
            need = int(L.mgr_rmsnorm_bwd_workspace_bytes(1 << 20, cols, code))
            assert 0 < need <= limit, f"{name} cols={cols}: {need} bytes of scratch exceed the fixed {limit}"
            if need > worst[0]:
                worst = (need, (name, cols))
    print(f"\n[largest scratch up to 16384 columns] {worst[0] / 2**20:.2f} MiB at {worst[1]}")
