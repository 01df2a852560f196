"""C-ABI checks that need no GPU: the library loads, exports every function include/mgr_b200.h
declares, and rejects bad arguments on the host before touching a device."""
import ctypes
import re
from pathlib import Path

import pytest

from mgrrmsnorm_b200 import _capi

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "mgr_b200.h"


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(mgr_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "mgr_rmsnorm_fwd" in names and "mgr_rmsnorm_bwd" in names and len(names) >= 8


def test_library_exports_every_declared_symbol(built_lib):
    raw = ctypes.CDLL(str(_capi.LIB_PATH))
    for name in declared_functions():
        assert hasattr(raw, name), f"libmgr_b200.so does not export {name}"


def test_python_signature_table_covers_header():
    assert sorted(_capi.SIGNATURES) == declared_functions()


def test_version_and_status_strings(built_lib):
    assert built_lib.mgr_abi_version() == 1
    assert _capi.status_str(0) == "ok"
    seen = set()
    for code in range(-10, 0):
        s = _capi.status_str(code)
        assert s and s != "unknown status" and s not in seen
        seen.add(s)
    assert _capi.status_str(-99) == "unknown status"


# Fake but well-aligned addresses: argument errors are reported before any pointer is dereferenced
# or any launch is attempted, so these calls are safe without a device.
P = 0x10000


@pytest.mark.parametrize("args,expect", [
    (dict(dtype=7), _capi.MGR_ERR_BAD_DTYPE),
    (dict(rows=-1), _capi.MGR_ERR_BAD_SHAPE),
    (dict(cols=0), _capi.MGR_ERR_BAD_SHAPE),
    (dict(cols=(1 << 30) + 1), _capi.MGR_ERR_TOO_LARGE),
    (dict(y=None), _capi.MGR_ERR_NULL_PTR),
    (dict(x=None), _capi.MGR_ERR_NULL_PTR),
    (dict(w=None), _capi.MGR_ERR_NULL_PTR),
    (dict(x=P + 2, dtype=_capi.MGR_F32), _capi.MGR_ERR_MISALIGNED),
    (dict(x=P + 1, dtype=_capi.MGR_F16), _capi.MGR_ERR_MISALIGNED),
    (dict(inv=P + 2), _capi.MGR_ERR_MISALIGNED),
    (dict(rows=0), _capi.MGR_OK),
])
def test_rmsnorm_fwd_argument_errors(built_lib, args, expect):
    a = dict(y=P, inv=P, x=P, w=P, rows=4, cols=64, eps=1e-5, dtype=_capi.MGR_F32)
    a.update(args)
    st = built_lib.mgr_rmsnorm_fwd(a["y"], a["inv"], a["x"], a["w"], a["rows"], a["cols"], a["eps"], a["dtype"], None)
    assert st == expect, _capi.status_str(st)


@pytest.mark.parametrize("args,expect", [
    (dict(dtype=-1), _capi.MGR_ERR_BAD_DTYPE),
    (dict(rows=-5), _capi.MGR_ERR_BAD_SHAPE),
    (dict(cols=-1), _capi.MGR_ERR_BAD_SHAPE),
    (dict(dw=None, dw32=None), _capi.MGR_ERR_NULL_PTR),
    (dict(dx=None), _capi.MGR_ERR_NULL_PTR),
    (dict(inv=None), _capi.MGR_ERR_NULL_PTR),
    (dict(ws=None), _capi.MGR_ERR_NULL_PTR),
    (dict(dy=P + 2), _capi.MGR_ERR_MISALIGNED),
    (dict(ws=P + 8), _capi.MGR_ERR_MISALIGNED),
    (dict(dw32=P + 1), _capi.MGR_ERR_MISALIGNED),
])
def test_rmsnorm_bwd_argument_errors(built_lib, args, expect):
    a = dict(dx=P, dw=P, dw32=None, dy=P, x=P, w=P, inv=P, rows=4, cols=64, dtype=_capi.MGR_F32, ws=P, wsb=1 << 20)
    a.update(args)
    st = built_lib.mgr_rmsnorm_bwd(a["dx"], a["dw"], a["dw32"], a["dy"], a["x"], a["w"], a["inv"], a["rows"], a["cols"],
                                   a["dtype"], a["ws"], a["wsb"], None)
    assert st == expect, _capi.status_str(st)


@pytest.mark.parametrize("fn", ["fwd", "bwd"])
def test_swiglu_act_argument_errors(built_lib, fn):
    def call(h=P, gv=P, dh=P, m=3, f=8, dtype=_capi.MGR_F16):
        if fn == "fwd":
            return built_lib.mgr_swiglu_act_fwd(h, gv, m, f, dtype, None)
        return built_lib.mgr_swiglu_act_bwd(h, dh, gv, m, f, dtype, None)

    assert call(dtype=3) == _capi.MGR_ERR_BAD_DTYPE
    assert call(m=-1) == _capi.MGR_ERR_BAD_SHAPE
    assert call(f=0) == _capi.MGR_ERR_BAD_SHAPE
    assert call(h=None) == _capi.MGR_ERR_NULL_PTR
    assert call(gv=None) == _capi.MGR_ERR_NULL_PTR
    assert call(gv=P + 1) == _capi.MGR_ERR_MISALIGNED
    assert call(m=0) == _capi.MGR_OK


def test_add_rmsnorm_argument_errors(built_lib):
    def fwd(y=P, h=P, inv=P, x=P, res=P, w=P, rows=4, cols=64, dtype=_capi.MGR_BF16):
        return built_lib.mgr_add_rmsnorm_fwd(y, h, inv, x, res, w, rows, cols, 1e-6, dtype, None)

    def bwd(dh=P, dw=P, dw32=None, dy=P, dres=P, h=P, w=P, inv=P, rows=4, cols=64, dtype=_capi.MGR_BF16, ws=P, wsb=1 << 20):
        return built_lib.mgr_add_rmsnorm_bwd(dh, dw, dw32, dy, dres, h, w, inv, rows, cols, dtype, ws, wsb, None)

    assert fwd(dtype=5) == _capi.MGR_ERR_BAD_DTYPE
    assert fwd(cols=0) == _capi.MGR_ERR_BAD_SHAPE
    assert fwd(res=None) == _capi.MGR_ERR_NULL_PTR          # the residual operand is required here
    assert fwd(h=None) == _capi.MGR_ERR_NULL_PTR
    assert fwd(res=P + 1) == _capi.MGR_ERR_MISALIGNED
    assert fwd(rows=0) == _capi.MGR_OK
    assert bwd(dtype=-2) == _capi.MGR_ERR_BAD_DTYPE
    assert bwd(rows=-1) == _capi.MGR_ERR_BAD_SHAPE
    assert bwd(dres=None) == _capi.MGR_ERR_NULL_PTR
    assert bwd(dw=None, dw32=None) == _capi.MGR_ERR_NULL_PTR
    assert bwd(dres=P + 1) == _capi.MGR_ERR_MISALIGNED
    assert bwd(ws=P + 4) == _capi.MGR_ERR_MISALIGNED


def test_gemm_family_argument_errors(built_lib):
    """Shape, dtype, pointer and pitch errors of the tensor-core entry points come back as status codes before
    any CUDA call is made."""
    L, F16 = built_lib, _capi.MGR_F16

    def gemm(c=P, a=P, b=P, m=16, n=64, k=64, lda=64, ldb=64, ldc=64, amn=0, bmn=0, dtype=F16):
        return L.mgr_gemm(c, a, b, m, n, k, lda, ldb, ldc, amn, bmn, dtype, None)

    assert gemm(dtype=_capi.MGR_F32) == _capi.MGR_ERR_BAD_DTYPE          # tensor-core kernels take fp16 / bf16 only
    assert gemm(n=60) == _capi.MGR_ERR_BAD_SHAPE and gemm(k=12) == _capi.MGR_ERR_BAD_SHAPE
    assert gemm(lda=32) == _capi.MGR_ERR_BAD_SHAPE                         # pitch shorter than the row
    assert gemm(ldc=68) == _capi.MGR_ERR_BAD_SHAPE                         # pitch not a multiple of 8 elements
    assert gemm(m=12, amn=1, lda=16) == _capi.MGR_ERR_BAD_SHAPE            # rows of an MN-major A are its inner dimension
    assert gemm(m=(1 << 30) + 8) == _capi.MGR_ERR_TOO_LARGE
    assert gemm(a=None) == _capi.MGR_ERR_NULL_PTR and gemm(c=P + 8) == _capi.MGR_ERR_MISALIGNED
    assert gemm(m=0) == _capi.MGR_OK
    assert L.mgr_gemm_tn(P, P, P, 16, 64, 63, 64, 64, 64, F16, None) == _capi.MGR_ERR_BAD_SHAPE
    for fn, nargs in ((L.mgr_swiglu_fused_fwd, 3), (L.mgr_swiglu_fused_bwd, 4), (L.mgr_swiglu_fused_fwd_save, 4), (L.mgr_swiglu_dh_dgv, 4)):
        ptrs = [P] * nargs
        assert fn(*ptrs, 16, 64, 64, _capi.MGR_F32, None) == _capi.MGR_ERR_BAD_DTYPE
        assert fn(*ptrs, 16, 64, 60, F16, None) == _capi.MGR_ERR_BAD_SHAPE
        assert fn(*ptrs, 16, 63, 64, F16, None) == _capi.MGR_ERR_BAD_SHAPE
        assert fn(*([None] + ptrs[1:]), 16, 64, 64, F16, None) == _capi.MGR_ERR_NULL_PTR
        assert fn(*([P + 2] + ptrs[1:]), 16, 64, 64, F16, None) == _capi.MGR_ERR_MISALIGNED
        assert fn(*ptrs, 0, 64, 64, F16, None) == _capi.MGR_OK
    assert L.mgr_gemm_set_sm_limit(0) >= 0            # returns the previous limit; 0 = all SMs
    assert L.mgr_gemm_set_sm_limit(100) == 0 and L.mgr_gemm_set_sm_limit(0) == 100


def test_workspace_query_rejects_bad_arguments(built_lib):
    assert built_lib.mgr_rmsnorm_bwd_workspace_bytes(-1, 64, _capi.MGR_F32) == 0
    assert built_lib.mgr_rmsnorm_bwd_workspace_bytes(4, 0, _capi.MGR_F32) == 0
    assert built_lib.mgr_rmsnorm_bwd_workspace_bytes(4, 64, 9) == 0


def test_no_device_is_reported_not_crashed(built_lib):
    import torch

    if torch.cuda.is_available():
        pytest.skip("a device is present")
    sms = ctypes.c_int(-1)
    assert built_lib.mgr_device_check(ctypes.byref(sms)) == _capi.MGR_ERR_CUDA
    st = built_lib.mgr_rmsnorm_fwd(P, P, P, P, 4, 64, 1e-5, _capi.MGR_F32, None)
    assert st == _capi.MGR_ERR_CUDA


def test_peer_allreduce_argument_errors(built_lib):
    """mgr_peer_allreduce_f32 checks its arguments on the host before anything is launched (no GPU needed)."""
    import ctypes

    L = built_lib
    assert L.mgr_peer_allreduce_buffer_bytes(2, 8192) == 2 * 2 * 8192 * 8      # [parity][sender][n] pairs of {value, call number}
    assert L.mgr_peer_allreduce_buffer_bytes(0, 8192) == 0 and L.mgr_peer_allreduce_buffer_bytes(17, 8192) == 0
    assert L.mgr_peer_allreduce_buffer_bytes(2, 6) == 0          # not a multiple of 4
    P = 0x10000
    bufs = (ctypes.c_void_p * 2)(P, P)
    call = lambda **kw: L.mgr_peer_allreduce_f32(kw.get("bufs", bufs), kw.get("rank", 0), kw.get("world", 2), kw.get("src", P),  # noqa: E731
                                                 kw.get("out32", P), kw.get("out", None), kw.get("dtype", _capi.MGR_BF16),
                                                 kw.get("n", 64), kw.get("n_max", 64), kw.get("calls", P), None)
    assert call(dtype=7) == _capi.MGR_ERR_BAD_DTYPE
    assert call(rank=2) == _capi.MGR_ERR_BAD_SHAPE and call(world=0) == _capi.MGR_ERR_BAD_SHAPE and call(world=17) == _capi.MGR_ERR_BAD_SHAPE
    assert call(n=6) == _capi.MGR_ERR_BAD_SHAPE and call(n=128, n_max=64) == _capi.MGR_ERR_BAD_SHAPE
    assert call(src=None) == _capi.MGR_ERR_NULL_PTR and call(calls=None) == _capi.MGR_ERR_NULL_PTR
    assert call(out32=None, out=None) == _capi.MGR_ERR_NULL_PTR
    assert call(bufs=(ctypes.c_void_p * 2)(P, None)) == _capi.MGR_ERR_NULL_PTR
    assert call(bufs=(ctypes.c_void_p * 2)(P, P + 16)) == _capi.MGR_ERR_MISALIGNED
    assert call(src=P + 4) == _capi.MGR_ERR_MISALIGNED
