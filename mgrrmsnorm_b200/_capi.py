"""ctypes view of libmgr_b200.so (declared in include/mgr_b200.h).

The library is the product; there is no fallback. If it has not been built, or cannot be loaded,
every access raises `MgrLibraryError` with the build command -- the same stance as the reference,
which raises "CUDA extension not compiled" at first use (megagemm/rmsnorm.py:23-24).
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libmgr_b200.so"

MGR_F32, MGR_F16, MGR_BF16 = 0, 1, 2
MGR_PEER_ALLREDUCE_CTAS = 16   # as in include/mgr_b200.h

MGR_OK = 0
MGR_ERR_BAD_DTYPE = -1
MGR_ERR_BAD_SHAPE = -2
MGR_ERR_NULL_PTR = -3
MGR_ERR_MISALIGNED = -4
MGR_ERR_WORKSPACE_TOO_SMALL = -5
MGR_ERR_UNSUPPORTED_ARCH = -6
MGR_ERR_LAUNCH_FAILED = -7
MGR_ERR_DEVICE_TIMEOUT = -8
MGR_ERR_TOO_LARGE = -9
MGR_ERR_CUDA = -10

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_int = ctypes.c_int
_f32 = ctypes.c_float
_sz = ctypes.c_size_t

# name -> (restype, argtypes); one entry per declaration in include/mgr_b200.h
SIGNATURES = {
    "mgr_abi_version": (_int, []),
    "mgr_status_str": (ctypes.c_char_p, [_int]),
    "mgr_reload_env": (None, []),
    "mgr_device_check": (_int, [ctypes.POINTER(_int)]),
    "mgr_device_status": (_int, [_int]),
    "mgr_debug_poke_device_status": (_int, [_int, _int]),
    "mgr_rmsnorm_fwd": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _f32, _int, _vp]),
    "mgr_rms_inv": (_int, [_vp, _vp, _i64, _i64, _f32, _int, _vp]),
    "mgr_rmsnorm_bwd_workspace_bytes": (_sz, [_i64, _i64, _int]),
    "mgr_rmsnorm_bwd": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _sz, _vp]),
    "mgr_rmsnorm_bwd_noalloc": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "mgr_add_rmsnorm_fwd": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _f32, _int, _vp]),
    "mgr_add_rmsnorm_bwd": (_int, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _int, _vp, _sz, _vp]),
    "mgr_swiglu_act_fwd": (_int, [_vp, _vp, _i64, _i64, _int, _vp]),
    "mgr_swiglu_act_bwd": (_int, [_vp, _vp, _vp, _i64, _i64, _int, _vp]),
    "mgr_swiglu_fused_fwd": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "mgr_swiglu_fused_fwd_scaled": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "mgr_gemm_tn": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _int, _vp]),
    "mgr_gemm": (_int, [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _int, _int, _int, _vp]),
    "mgr_swiglu_fused_bwd": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "mgr_swiglu_fused_fwd_save": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "mgr_swiglu_dh_dgv": (_int, [_vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp]),
    "mgr_gemm_set_sm_limit": (_int, [_int]),
    "mgr_peer_allreduce_buffer_bytes": (_sz, [_int, _i64]),
    "mgr_peer_allreduce_f32": (_int, [_vp, _int, _int, _vp, _vp, _vp, _int, _i64, _i64, _vp, _vp]),
}


class MgrLibraryError(RuntimeError):
    pass


class MgrStatusError(RuntimeError):
    """A C-ABI call returned a non-zero status."""

    def __init__(self, fn: str, status: int, text: str):
        super().__init__(f"{fn} failed: {text} (status {status})")
        self.status = status


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library with argtypes/restypes set. Raises MgrLibraryError if it is not there."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise MgrLibraryError(
            f"{LIB_PATH} is missing: the sm_100a kernel library has not been built. "
            "Run `python -m mgrrmsnorm_b200.build` (needs nvcc). There is no CPU or PyTorch fallback.")
    try:
        L = ctypes.CDLL(str(LIB_PATH))
    except OSError as e:  # pragma: no cover - depends on the machine
        raise MgrLibraryError(f"cannot load {LIB_PATH}: {e}") from e
    for name, (res, args) in SIGNATURES.items():
        try:
            fn = getattr(L, name)
        except AttributeError as e:
            raise MgrLibraryError(f"{LIB_PATH} does not export {name}; rebuild it") from e
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L


def reload_env() -> None:
    """Makes the library read the MGR_* environment overrides again (it reads them once, at first use)."""
    lib().mgr_reload_env()


def status_str(status: int) -> str:
    return lib().mgr_status_str(int(status)).decode()


def check(fn: str, status: int) -> None:
    if status != MGR_OK:
        raise MgrStatusError(fn, status, status_str(status))
