"""Host-side mirror of the reference's operator API: names, shapes, state-dict layout, error
behaviour. CPU only (no kernel is launched)."""
import numpy as np
import pytest
import torch


def test_package_exports_are_lazy_and_complete():
    import mgrrmsnorm_b200 as pkg

    reference_names = {"RMSNorm", "RMSNormFunction", "MegaGemmTriton", "MegaGemmFunction", "__version__"}
    # not in the reference: the residual add fused into the norm, and the norm folded into the projection
    added = {"AddRMSNorm", "AddRMSNormFunction", "PreNormSwiGLU"}
    assert set(pkg.__all__) == reference_names | added
    for name in sorted((reference_names | added) - {"__version__"}):
        assert getattr(pkg, name).__name__ == name
    with pytest.raises(AttributeError):
        pkg.NoSuchThing


def test_reference_import_paths_resolve():
    import megagemm
    import rmsnorm_cuda_ops
    from megagemm import MegaGemmTriton, RMSNorm  # noqa: F401
    from megagemm.rmsnorm import RMSNormFunction  # noqa: F401
    from megagemm.swiglu import MegaGemmFunction  # noqa: F401

    assert megagemm.__version__ == "0.1.0"
    assert callable(rmsnorm_cuda_ops.rmsnorm_forward) and callable(rmsnorm_cuda_ops.rmsnorm_backward)


def test_rmsnorm_module_surface():
    from mgrrmsnorm_b200 import RMSNorm

    m = RMSNorm(4096)
    assert m.epsilon == 1e-5 and m.hidden_size == 4096
    assert list(m.state_dict()) == ["weight"] and m.weight.shape == (4096,) and m.weight.dtype == torch.float32
    assert torch.all(m.weight == 1)
    assert repr(m) == "RMSNorm(hidden_size=4096, eps=1e-05)"
    assert RMSNorm(8, epsilon=1e-6).epsilon == 1e-6


def test_swiglu_module_surface_and_hidden_rule(golden_dir):
    from mgrrmsnorm_b200 import MegaGemmTriton

    rule = np.load(golden_dir / "swiglu.npz")["hidden_rule"]
    for dm, mo, hm, hidden in rule:
        m = MegaGemmTriton(int(dm), multiple_of=int(mo), hidden_multiple=float(hm))
        assert m.hidden == int(hidden)
        assert tuple(m.w12.weight.shape) == (2 * int(hidden), int(dm))
        assert tuple(m.w3.weight.shape) == (int(dm), int(hidden))
        assert m.w12.bias is None and m.w3.bias is None
    assert sorted(MegaGemmTriton(64, 32).state_dict()) == ["w12.weight", "w3.weight"]
    assert MegaGemmTriton(4096).hidden == 6912
    assert MegaGemmTriton(8192, hidden_multiple=3.5).hidden == 28672


def test_reference_state_dict_loads(golden_dir):
    from mgrrmsnorm_b200 import MegaGemmTriton

    g = np.load(golden_dir / "swiglu.npz")
    m = MegaGemmTriton(64, multiple_of=32)
    m.load_state_dict({"w12.weight": torch.from_numpy(g["mlp_w12"]), "w3.weight": torch.from_numpy(g["mlp_w3"])})


def test_cpu_tensors_are_refused_like_the_reference():
    import rmsnorm_cuda_ops as ops

    x = torch.randn(4, 8)
    w = torch.ones(8)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ops.rmsnorm_forward(x, w, 1e-5)
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ops.rmsnorm_backward(x, x, w, torch.ones(4))
    with pytest.raises(RuntimeError, match="must be a CUDA tensor"):
        ops.swiglu_act_forward(x, 4)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from mgrrmsnorm_b200 import _capi

    monkeypatch.setattr(_capi, "_lib", None)
    monkeypatch.setattr(_capi, "LIB_PATH", tmp_path / "libmgr_b200.so")
    with pytest.raises(_capi.MgrLibraryError, match="no CPU or PyTorch fallback"):
        _capi.lib()
