"""CPU oracle for the two MegaGemm hot paths (RMSNorm, SwiGLU MLP).

TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared with. Nothing in the product
package imports this module; only tests/, the smoke check and the benchmark's CPU-baseline leg do.

Three layers, each citing the reference lines it restates:
  * `lib()`           -- ctypes view of oracle/lib/libmgr_oracle.so (mgr_oracle.c): fp64 ground truth
                         and the reference's fp32 CPU evaluation order for the forward;
  * numpy wrappers    -- `rmsnorm_fwd`, `rmsnorm_bwd`, `swiglu_act_fwd`, `swiglu_act_bwd`, `swiglu_mlp`;
  * torch formulas    -- `rmsnorm_formula_torch` (test_rmsnorm.py:55-60) and `swiglu_formula_torch`
                         (PyTorchSwiGLU, benchmark_swiglu.py:40-58), used as the timed CPU baseline.
`ref_lib()` opens oracle/_ref/libmgr_ref.so when present: the reference's own sources compiled
unmodified (its CPU forward and its six CUDA wrappers built for sm_100a).

Parity is pinned: tests/test_oracle_golden.py checks these functions against vectors produced by the
reference's own code (rmsnorm_cpu; its Triton kernels run under the Triton interpreter; its torch
modules), stored under tests/golden/.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "lib" / "libmgr_oracle.so"
REF_LIB_PATH = HERE / "_ref" / "libmgr_ref.so"

_lib = None
_ref = None

_i64 = ctypes.c_int64
_f32 = ctypes.c_float
_ptr = ctypes.c_void_p


def build(with_ref: bool = True) -> None:
    """Runs oracle/Makefile (gcc for the restatement; nvcc over the reference tree when it is mounted)."""
    targets = ["liboracle"] + (["ref"] if with_ref else [])
    subprocess.run(["make", "-C", str(HERE), *targets], check=True, capture_output=True)


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build(with_ref=False)
        L = ctypes.CDLL(str(LIB_PATH))
        L.mgr_oracle_threads.restype = ctypes.c_int
        L.mgr_oracle_rmsnorm_fwd_f64.argtypes = [_ptr, _ptr, _ptr, _ptr, _i64, _i64, _f32]
        L.mgr_oracle_rmsnorm_fwd_f32seq.argtypes = [_ptr, _ptr, _ptr, _i64, _i64, _f32]
        L.mgr_oracle_rmsnorm_bwd_f64.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _i64, _i64, _f32]
        L.mgr_oracle_swiglu_act_fwd_f64.argtypes = [_ptr, _ptr, _i64, _i64]
        L.mgr_oracle_swiglu_act_bwd_f64.argtypes = [_ptr, _ptr, _ptr, _i64, _i64]
        L.mgr_oracle_linear_f64.argtypes = [_ptr, _ptr, _ptr, _i64, _i64, _i64]
        for fn in ("mgr_oracle_rmsnorm_fwd_f64", "mgr_oracle_rmsnorm_fwd_f32seq", "mgr_oracle_rmsnorm_bwd_f64",
                   "mgr_oracle_swiglu_act_fwd_f64", "mgr_oracle_swiglu_act_bwd_f64", "mgr_oracle_linear_f64"):
            getattr(L, fn).restype = None
        _lib = L
    return _lib


def threads() -> int:
    return int(lib().mgr_oracle_threads())


def _f32c(a) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32))


def _p(a: np.ndarray) -> int:
    return a.ctypes.data


# ---------------------------------------------------------------------------------------------------
# dtype helpers: the oracle works on fp32 arrays holding values already rounded to the test dtype
# ---------------------------------------------------------------------------------------------------

def round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    """Rounds to `dtype` ('f32' | 'f16' | 'bf16', round-to-nearest-even) and returns the values as fp32."""
    a = np.asarray(a, dtype=np.float32)
    if dtype == "f32":
        return a.copy()
    if dtype == "f16":
        return a.astype(np.float16).astype(np.float32)
    if dtype == "bf16":
        u = a.view(np.uint32).astype(np.uint64)
        rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        nan = np.isnan(a)
        out = rounded.astype(np.uint32).view(np.float32).reshape(a.shape).copy()
        out[nan] = np.nan
        return out
    raise ValueError(dtype)


def ulp_of(a: np.ndarray, dtype: str) -> np.ndarray:
    """Spacing of `dtype` at |a| (one unit in the last place of the output type)."""
    mant = {"f32": 23, "f16": 10, "bf16": 7}[dtype]
    emin = {"f32": -126, "f16": -14, "bf16": -126}[dtype]
    mag = np.abs(np.asarray(a, dtype=np.float64))
    e = np.floor(np.log2(np.maximum(mag, 2.0 ** emin)))
    return 2.0 ** (e - mant)


# ---------------------------------------------------------------------------------------------------
# numpy wrappers over the C restatement
# ---------------------------------------------------------------------------------------------------

def rmsnorm_fwd(x, w, eps: float):
    """fp64 truth: returns (y [R,H] float64, inv_rms [R] float64). src/rmsnorm_kernel.cu:56-101."""
    x = _f32c(x); w = _f32c(w)
    rows, cols = x.shape
    y = np.empty((rows, cols), np.float64); inv = np.empty(rows, np.float64)
    lib().mgr_oracle_rmsnorm_fwd_f64(_p(y), _p(inv), _p(x), _p(w), rows, cols, np.float32(eps))
    return y, inv


def rmsnorm_fwd_f32seq(x, w, eps: float) -> np.ndarray:
    """The reference's CPU evaluation order in fp32 (rmsnorm_standalone.cu:17-30)."""
    x = _f32c(x); w = _f32c(w)
    rows, cols = x.shape
    y = np.empty((rows, cols), np.float32)
    lib().mgr_oracle_rmsnorm_fwd_f32seq(_p(y), _p(x), _p(w), rows, cols, np.float32(eps))
    return y


def rmsnorm_bwd(dy, x, w, eps: float):
    """fp64 truth: returns (dx [R,H] float64, dw [H] float64). src/rmsnorm_kernel.cu:258-312."""
    dy = _f32c(dy); x = _f32c(x); w = _f32c(w)
    rows, cols = x.shape
    dx = np.empty((rows, cols), np.float64); dw = np.empty(cols, np.float64)
    lib().mgr_oracle_rmsnorm_bwd_f64(_p(dx), _p(dw), _p(dy), _p(x), _p(w), rows, cols, np.float32(eps))
    return dx, dw


def swiglu_act_fwd(gv, f: int) -> np.ndarray:
    """h = silu(gate)*val for gv = [gate | val] of shape [M, 2F]. megagemm/swiglu.py:35-41."""
    gv = _f32c(gv)
    m = gv.shape[0]
    h = np.empty((m, f), np.float64)
    lib().mgr_oracle_swiglu_act_fwd_f64(_p(h), _p(gv), m, f)
    return h


def swiglu_act_bwd(dh, gv, f: int) -> np.ndarray:
    """[d_gate | d_val] of shape [M, 2F]. megagemm/swiglu.py:64-76."""
    dh = _f32c(dh); gv = _f32c(gv)
    m = gv.shape[0]
    dgv = np.empty((m, 2 * f), np.float64)
    lib().mgr_oracle_swiglu_act_bwd_f64(_p(dgv), _p(dh), _p(gv), m, f)
    return dgv


def linear(a, b) -> np.ndarray:
    """a [M,K] x b[N,K]^T in fp64 (nn.Linear without bias, megagemm/swiglu.py:163-169)."""
    return np.asarray(a, np.float64) @ np.asarray(b, np.float64).T


def swiglu_mlp(x, w12, w3, dy=None, round_intermediates: str | None = None):
    """SwiGLU MLP forward (and backward when dy is given) in fp64.

    y = w3( silu(x w12[:F]^T) * (x w12[F:]^T) ): megagemm/swiglu.py:166-169 with the gate/value row
    layout of benchmark_swiglu.py:85-89. `round_intermediates` ('f16'/'bf16') rounds w12_out and h to
    that dtype as the reference's two-step path does (its nn.Linear and Triton kernel each store in
    the input dtype); None keeps them in fp64 (what a fused epilogue computes).
    Returns dict(y, h, gv[, dx, dw12, dw3]).
    """
    x = np.asarray(x, np.float64); w12 = np.asarray(w12, np.float64); w3 = np.asarray(w3, np.float64)
    f = w3.shape[1]
    gv = x @ w12.T
    if round_intermediates:
        gv = round_to(gv, round_intermediates).astype(np.float64)
    h = swiglu_act_fwd(gv, f) if round_intermediates else _act_fwd_f64(gv, f)
    if round_intermediates:
        h = round_to(h, round_intermediates).astype(np.float64)
    y = h @ w3.T
    out = {"y": y, "h": h, "gv": gv}
    if dy is not None:
        dy = np.asarray(dy, np.float64)
        dh = dy @ w3
        out["dw3"] = dy.T @ h
        dgv = _act_bwd_f64(dh, gv, f)
        out["dgv"] = dgv
        out["dx"] = dgv @ w12
        out["dw12"] = dgv.T @ x
    return out


def _act_fwd_f64(gv: np.ndarray, f: int) -> np.ndarray:
    g, v = gv[:, :f], gv[:, f:]
    return g / (1.0 + np.exp(-g)) * v


def _act_bwd_f64(dh: np.ndarray, gv: np.ndarray, f: int) -> np.ndarray:
    g, v = gv[:, :f], gv[:, f:]
    sig = 1.0 / (1.0 + np.exp(-g))
    return np.concatenate([dh * v * sig * (1.0 + g * (1.0 - sig)), dh * g * sig], axis=1)


# ---------------------------------------------------------------------------------------------------
# torch formulas (the reference's CPU path; also the timed CPU baseline)
# ---------------------------------------------------------------------------------------------------

def rmsnorm_formula_torch(x, w, eps: float, dy=None):
    """y = x * rsqrt(mean(x^2, -1) + eps) * w with autograd backward: test_rmsnorm.py:55-60.
    Tensors may be any float dtype on CPU. Returns (y, dx, dw); dx/dw are None without dy."""
    import torch

    x = x.detach().clone().requires_grad_(dy is not None)
    w = w.detach().clone().requires_grad_(dy is not None)
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w
    if dy is None:
        return y.detach(), None, None
    y.backward(dy)
    return y.detach(), x.grad, w.grad


def swiglu_formula_torch(x, w12, w3, dy=None):
    """w3(silu(w1 x) * (w2 x)) with w1 = w12[:F], w2 = w12[F:]: benchmark_swiglu.py:40-58, 85-89."""
    import torch
    import torch.nn.functional as F

    f = w3.shape[1]
    leaves = [t.detach().clone().requires_grad_(dy is not None) for t in (x, w12, w3)]
    xx, ww12, ww3 = leaves
    y = F.linear(F.silu(F.linear(xx, ww12[:f])) * F.linear(xx, ww12[f:]), ww3)
    if dy is None:
        return y.detach(), None, None, None
    y.backward(dy)
    return y.detach(), xx.grad, ww12.grad, ww3.grad


# ---------------------------------------------------------------------------------------------------
# the reference's own compiled sources (oracle/_ref), when present
# ---------------------------------------------------------------------------------------------------

_REF_SYMBOLS = {
    # C++-mangled names of the reference's functions (Itanium ABI), from its unmodified sources
    "rmsnorm_cpu": "_Z11rmsnorm_cpuPfPKfS1_iif",                                   # rmsnorm_standalone.cu:17
    "fwd_f32": "_Z17rmsnorm_cuda_fp32PfS_PKfS1_iif",                               # src/rmsnorm_kernel.cu:529
    "fwd_f16": "_Z17rmsnorm_cuda_fp16P6__halfPfPKS_S3_iif",                        # :577
    "fwd_bf16": "_Z17rmsnorm_cuda_bf16P13__nv_bfloat16PfPKS_S3_iif",               # :621
    "bwd_f32": "_Z26rmsnorm_backward_cuda_fp32PfS_PKfS1_S1_S1_ii",                 # :552
    "bwd_f16": "_Z26rmsnorm_backward_cuda_fp16P6__halfS0_PKS_S2_S2_PKfii",         # :596
    "bwd_bf16": "_Z26rmsnorm_backward_cuda_bf16P13__nv_bfloat16S0_PKS_S2_S2_PKfii",  # :640
}


class RefLib:
    """The reference's compiled functions. CUDA wrappers take device pointers and launch on the legacy
    default stream (the caller synchronises)."""

    def __init__(self, cdll: ctypes.CDLL):
        self._l = cdll
        self.rmsnorm_cpu = getattr(cdll, _REF_SYMBOLS["rmsnorm_cpu"])
        self.rmsnorm_cpu.argtypes = [_ptr, _ptr, _ptr, ctypes.c_int, ctypes.c_int, _f32]
        self.rmsnorm_cpu.restype = None
        self.fwd = {}
        self.bwd = {}
        for dt in ("f32", "f16", "bf16"):
            f = getattr(cdll, _REF_SYMBOLS["fwd_" + dt])
            f.argtypes = [_ptr, _ptr, _ptr, _ptr, ctypes.c_int, ctypes.c_int, _f32]
            f.restype = ctypes.c_bool
            b = getattr(cdll, _REF_SYMBOLS["bwd_" + dt])
            b.argtypes = [_ptr, _ptr, _ptr, _ptr, _ptr, _ptr, ctypes.c_int, ctypes.c_int]
            b.restype = ctypes.c_bool
            self.fwd[dt] = f
            self.bwd[dt] = b

    def cpu_forward(self, x, w, eps: float) -> np.ndarray:
        x = _f32c(x); w = _f32c(w)
        y = np.empty_like(x)
        self.rmsnorm_cpu(_p(y), _p(x), _p(w), x.shape[0], x.shape[1], np.float32(eps))
        return y


def ref_lib():
    """RefLib over oracle/_ref/libmgr_ref.so, or None when it was never built (no reference tree)."""
    global _ref
    if _ref is None:
        if not REF_LIB_PATH.exists():
            return None
        try:
            _ref = RefLib(ctypes.CDLL(str(REF_LIB_PATH)))
        except OSError:
            return None
    return _ref
