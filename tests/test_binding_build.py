"""The compiled torch extension (pytorch_binding/binding.cpp -> mgrrmsnorm_b200/pybind/rmsnorm_cuda_ops*.so):
it builds on a machine without a GPU, exports the reference binding's two functions (binding.cpp:136-139)
plus the rest of the operator surface, and refuses bad arguments with the reference's messages before
anything would be launched."""
import pytest
import torch


@pytest.fixture(scope="module")
def ext(built_lib):
    from mgrrmsnorm_b200 import build

    path = build.build_binding()          # incremental; compiles with torch's BuildExtension on first use
    assert path.exists() and path.parent.name == "pybind"
    from mgrrmsnorm_b200.pybind import rmsnorm_cuda_ops

    return rmsnorm_cuda_ops


def test_exports_the_whole_operator_surface(ext):
    import mgrrmsnorm_b200.rmsnorm_cuda_ops as ops

    for name in ops.ENTRY_POINTS:
        assert callable(getattr(ext, name)), name
        assert callable(ops.ctypes_impl[name]), name
    assert callable(ext.device_status) and callable(ext.set_gemm_sm_limit)


def test_python_layer_prefers_the_compiled_binding(ext, monkeypatch):
    import importlib

    import mgrrmsnorm_b200.rmsnorm_cuda_ops as ops

    ops = importlib.reload(ops)
    assert ops.BINDING == "pybind" and ops.rmsnorm_forward is ext.rmsnorm_forward
    monkeypatch.setenv("MGR_BINDING", "ctypes")
    ops = importlib.reload(ops)
    assert ops.BINDING == "ctypes" and ops.rmsnorm_forward is ops.ctypes_impl["rmsnorm_forward"]
    monkeypatch.delenv("MGR_BINDING")
    importlib.reload(ops)


@pytest.mark.parametrize("route", ["pybind", "ctypes"])
def test_argument_checks_match_the_reference_binding(ext, route):
    """CHECK_CUDA / CHECK_CONTIGUOUS texts of binding.cpp:9-11, raised as RuntimeError (TORCH_CHECK)."""
    import mgrrmsnorm_b200.rmsnorm_cuda_ops as ops

    fn = (lambda n: getattr(ext, n)) if route == "pybind" else (lambda n: ops.ctypes_impl[n])
    x, w = torch.zeros(4, 8), torch.ones(8)
    with pytest.raises(RuntimeError, match="input must be a CUDA tensor"):
        fn("rmsnorm_forward")(x, w, 1e-6)
    with pytest.raises(RuntimeError, match="grad_output must be a CUDA tensor"):
        fn("rmsnorm_backward")(x, x, w, torch.zeros(4))
    with pytest.raises(RuntimeError, match="w12_out must be a CUDA tensor"):
        fn("swiglu_act_forward")(torch.zeros(4, 16), 8)
    with pytest.raises(RuntimeError, match="a must be a CUDA tensor"):
        fn("gemm")(x, x, False, False)


def test_set_gemm_sm_limit_round_trip(ext, built_lib):
    """Host-only setting shared by both routes: the extension and ctypes talk to the same loaded library."""
    prev = ext.set_gemm_sm_limit(132)
    assert built_lib.mgr_gemm_set_sm_limit(prev) == 132
