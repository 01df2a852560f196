"""`rmsnorm_cuda_ops`: the extension module the reference's Python layer imports, on the new C ABI.

Same Python-visible surface as pytorch_binding/binding.cpp:136-139:
    rmsnorm_forward(input[R,H], weight[H], epsilon) -> [output[R,H], inv_rms[R] fp32]
    rmsnorm_backward(grad_output[R,H], input[R,H], weight[H], inv_rms[R]) -> [grad_input, grad_weight]
and the same duties as that binding: check the tensors (binding.cpp:9-11,17-24,79-82), allocate the
outputs through torch (:29-30, :89-90), dispatch on the input dtype (:34-63, :94-129), raise
RuntimeError on failure (:65, :131). Added, because the reference lacks them: a device guard and a
launch on torch's current stream (the reference launches on the legacy default stream of whichever
device is current, src/rmsnorm_kernel.cu:542,564).

torch is used for device memory and streams only; all arithmetic is in libmgr_b200.so.

Two routes to the same C ABI: the functions below (ctypes, need no compiler beyond the one that built the
library), and the compiled torch extension built from pytorch_binding/binding.cpp by setup.py, which has
the same functions with less per-call overhead. When the extension is present in mgrrmsnorm_b200/pybind/ it
replaces the functions listed in `ENTRY_POINTS` at import (`BINDING` says which route is active;
MGR_BINDING=ctypes keeps the ctypes route). The ctypes versions stay reachable as `ctypes_impl[name]`.
"""
from __future__ import annotations

import os

import torch

from . import _capi

_DTYPES = {torch.float32: _capi.MGR_F32, torch.float16: _capi.MGR_F16, torch.bfloat16: _capi.MGR_BF16}


def _check_input(t: torch.Tensor, name: str) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def _dtype_code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise RuntimeError(f"Unsupported dtype{what}. Use float32, float16, or bfloat16.") from None


def _stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _out_or_new(out, shape, like: torch.Tensor, name: str) -> torch.Tensor:
    """`out` checked as a contiguous tensor of `shape` with `like`'s dtype and device (e.g. a row slab of a
    larger buffer), or a new tensor when it is None."""
    if out is None:
        return torch.empty(shape, device=like.device, dtype=like.dtype)
    if tuple(out.shape) != tuple(shape) or out.dtype != like.dtype or out.device != like.device or not out.is_contiguous():
        raise RuntimeError(f"{name} must be a contiguous {list(shape)} tensor of the operands' dtype and device")
    return out


def rmsnorm_forward(input: torch.Tensor, weight: torch.Tensor, epsilon: float):
    """[output, inv_rms] = RMSNorm forward of a 2-D tensor (binding.cpp:16-68)."""
    _check_input(input, "input")
    _check_input(weight, "weight")
    if input.dim() != 2:
        raise RuntimeError("Input must be 2D")
    rows, cols = input.shape
    if weight.dim() != 1 or weight.shape[0] != cols:
        raise RuntimeError("Weight size must match hidden size")
    code = _dtype_code(input, "")
    if weight.dtype != input.dtype:
        # binding.cpp:48,57: weight.data_ptr<T>() throws when the dtypes differ
        raise RuntimeError(f"weight dtype {weight.dtype} must match input dtype {input.dtype}")
    if weight.device != input.device:
        raise RuntimeError("input and weight must be on the same device")
    L = _capi.lib()
    with torch.cuda.device(input.device):
        inv_rms = torch.empty((rows,), dtype=torch.float32, device=input.device)
        output = torch.empty_like(input)
        st = L.mgr_rmsnorm_fwd(output.data_ptr(), inv_rms.data_ptr(), input.data_ptr(), weight.data_ptr(),
                               rows, cols, float(epsilon), code, _stream_ptr(input.device))
    _capi.check("RMSNorm Forward CUDA kernel", st)
    return [output, inv_rms]


def rms_inv(input: torch.Tensor, epsilon: float) -> torch.Tensor:
    """inv_rms[R] (fp32) of a 2-D tensor alone: the forward's row scales without its output (one read of the
    input). Same bits as the inv_rms rmsnorm_forward returns."""
    _check_input(input, "input")
    if input.dim() != 2:
        raise RuntimeError("Input must be 2D")
    rows, cols = input.shape
    code = _dtype_code(input, "")
    L = _capi.lib()
    with torch.cuda.device(input.device):
        inv_rms = torch.empty((rows,), dtype=torch.float32, device=input.device)
        st = L.mgr_rms_inv(inv_rms.data_ptr(), input.data_ptr(), rows, cols, float(epsilon), code, _stream_ptr(input.device))
    _capi.check("RMSNorm row-scale CUDA kernel", st)
    return inv_rms


def rmsnorm_backward_full(grad_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor,
                          inv_rms: torch.Tensor, want_dw_f32: bool = False):
    """[grad_input, grad_weight, grad_weight_fp32 | None]; the fp32 sum is what a row-sharded caller
    all-reduces before rounding."""
    for t, n in ((grad_output, "grad_output"), (input, "input"), (weight, "weight"), (inv_rms, "inv_rms")):
        _check_input(t, n)
    if input.dim() != 2:
        raise RuntimeError("Input must be 2D")
    rows, cols = input.shape
    if grad_output.shape != input.shape:
        raise RuntimeError("grad_output shape must match input shape")
    if weight.dim() != 1 or weight.shape[0] != cols:
        raise RuntimeError("Weight size must match hidden size")
    if inv_rms.dtype != torch.float32 or inv_rms.numel() != rows:
        raise RuntimeError("inv_rms must be a float32 tensor with one value per row")
    code = _dtype_code(input, " for backward")
    if grad_output.dtype != input.dtype or weight.dtype != input.dtype:
        raise RuntimeError("grad_output, input and weight must share one dtype")
    if not (grad_output.device == input.device == weight.device == inv_rms.device):
        raise RuntimeError("all tensors must be on the same device")
    L = _capi.lib()
    with torch.cuda.device(input.device):
        grad_input = torch.empty_like(input)
        grad_weight = torch.empty_like(weight)
        dw_f32 = torch.empty((cols,), dtype=torch.float32, device=input.device) if want_dw_f32 else None
        ws_bytes = int(L.mgr_rmsnorm_bwd_workspace_bytes(rows, cols, code))
        ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=input.device)
        st = L.mgr_rmsnorm_bwd(grad_input.data_ptr(), grad_weight.data_ptr(),
                               dw_f32.data_ptr() if dw_f32 is not None else None,
                               grad_output.data_ptr(), input.data_ptr(), weight.data_ptr(), inv_rms.data_ptr(),
                               rows, cols, code, ws.data_ptr(), ws.numel(), _stream_ptr(input.device))
    _capi.check("RMSNorm Backward CUDA kernel", st)
    return [grad_input, grad_weight, dw_f32]


def rmsnorm_backward(grad_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, inv_rms: torch.Tensor):
    """[grad_input, grad_weight] (binding.cpp:73-134). grad_weight has the weight's dtype, as there."""
    return rmsnorm_backward_full(grad_output, input, weight, inv_rms)[:2]


def add_rmsnorm_forward(input: torch.Tensor, residual: torch.Tensor, weight: torch.Tensor, epsilon: float,
                        inplace: bool = False):
    """[output, hidden, inv_rms] with hidden = input + residual and output = RMSNorm(hidden) * weight.

    One kernel for the `h = x + residual; y = norm(h)` pair that opens a pre-norm block; the same bits as
    the torch add followed by rmsnorm_forward. `inplace=True` writes hidden over `residual` (the residual
    stream is updated where it lies) and returns that tensor.
    """
    _check_input(input, "input")
    _check_input(residual, "residual")
    _check_input(weight, "weight")
    if input.dim() != 2:
        raise RuntimeError("Input must be 2D")
    rows, cols = input.shape
    if residual.shape != input.shape:
        raise RuntimeError("residual shape must match input shape")
    if weight.dim() != 1 or weight.shape[0] != cols:
        raise RuntimeError("Weight size must match hidden size")
    code = _dtype_code(input, "")
    if weight.dtype != input.dtype or residual.dtype != input.dtype:
        raise RuntimeError("input, residual and weight must share one dtype")
    if not (input.device == residual.device == weight.device):
        raise RuntimeError("all tensors must be on the same device")
    L = _capi.lib()
    with torch.cuda.device(input.device):
        inv_rms = torch.empty((rows,), dtype=torch.float32, device=input.device)
        output = torch.empty_like(input)
        hidden = residual if inplace else torch.empty_like(input)
        st = L.mgr_add_rmsnorm_fwd(output.data_ptr(), hidden.data_ptr(), inv_rms.data_ptr(), input.data_ptr(),
                                   residual.data_ptr(), weight.data_ptr(), rows, cols, float(epsilon), code,
                                   _stream_ptr(input.device))
    _capi.check("Add+RMSNorm Forward CUDA kernel", st)
    return [output, hidden, inv_rms]


def add_rmsnorm_backward(grad_output: torch.Tensor, grad_hidden: torch.Tensor, hidden: torch.Tensor,
                         weight: torch.Tensor, inv_rms: torch.Tensor, want_dw_f32: bool = False):
    """[grad_hidden_total, grad_weight, grad_weight_fp32 | None]: the norm's input gradient plus the
    gradient that arrives along the residual stream, rounded once. It is the gradient of both `input`
    and `residual` of add_rmsnorm_forward."""
    for t, n in ((grad_output, "grad_output"), (grad_hidden, "grad_hidden"), (hidden, "hidden"), (weight, "weight"),
                 (inv_rms, "inv_rms")):
        _check_input(t, n)
    if hidden.dim() != 2:
        raise RuntimeError("Input must be 2D")
    rows, cols = hidden.shape
    if grad_output.shape != hidden.shape or grad_hidden.shape != hidden.shape:
        raise RuntimeError("gradient shapes must match the hidden shape")
    if weight.dim() != 1 or weight.shape[0] != cols:
        raise RuntimeError("Weight size must match hidden size")
    if inv_rms.dtype != torch.float32 or inv_rms.numel() != rows:
        raise RuntimeError("inv_rms must be a float32 tensor with one value per row")
    code = _dtype_code(hidden, " for backward")
    if not (grad_output.dtype == grad_hidden.dtype == weight.dtype == hidden.dtype):
        raise RuntimeError("grad_output, grad_hidden, hidden and weight must share one dtype")
    if not (grad_output.device == grad_hidden.device == hidden.device == weight.device == inv_rms.device):
        raise RuntimeError("all tensors must be on the same device")
    L = _capi.lib()
    with torch.cuda.device(hidden.device):
        grad_total = torch.empty_like(hidden)
        grad_weight = torch.empty_like(weight)
        dw_f32 = torch.empty((cols,), dtype=torch.float32, device=hidden.device) if want_dw_f32 else None
        ws_bytes = int(L.mgr_rmsnorm_bwd_workspace_bytes(rows, cols, code))
        ws = torch.empty((max(ws_bytes, 16),), dtype=torch.uint8, device=hidden.device)
        st = L.mgr_add_rmsnorm_bwd(grad_total.data_ptr(), grad_weight.data_ptr(),
                                   dw_f32.data_ptr() if dw_f32 is not None else None,
                                   grad_output.data_ptr(), grad_hidden.data_ptr(), hidden.data_ptr(), weight.data_ptr(),
                                   inv_rms.data_ptr(), rows, cols, code, ws.data_ptr(), ws.numel(),
                                   _stream_ptr(hidden.device))
    _capi.check("Add+RMSNorm Backward CUDA kernel", st)
    return [grad_total, grad_weight, dw_f32]


# ---------------------------------------------------------------------------------------------------
# SwiGLU entry points. The reference has no native code here (its activation is a Triton kernel inside
# megagemm/swiglu.py); these are what that file calls instead.
# ---------------------------------------------------------------------------------------------------

def swiglu_act_forward(w12_out: torch.Tensor, hidden_dim: int) -> torch.Tensor:
    """h[M, hidden] = silu(w12_out[:, :hidden]) * w12_out[:, hidden:] for a contiguous [M, 2*hidden]
    tensor (the launch in megagemm/swiglu.py:96-107)."""
    _check_input(w12_out, "w12_out")
    if w12_out.dim() != 2 or w12_out.shape[1] != 2 * hidden_dim:
        raise RuntimeError("w12_out must be [M, 2*hidden_dim]")
    code = _dtype_code(w12_out, "")
    m = w12_out.shape[0]
    L = _capi.lib()
    with torch.cuda.device(w12_out.device):
        out = torch.empty((m, hidden_dim), device=w12_out.device, dtype=w12_out.dtype)
        st = L.mgr_swiglu_act_fwd(out.data_ptr(), w12_out.data_ptr(), m, hidden_dim, code, _stream_ptr(w12_out.device))
    _capi.check("SwiGLU activation forward kernel", st)
    return out


def swiglu_act_backward(grad_out: torch.Tensor, w12_out: torch.Tensor, hidden_dim: int) -> torch.Tensor:
    """[d_gate | d_val] of shape [M, 2*hidden] (the launch in megagemm/swiglu.py:116-129)."""
    _check_input(grad_out, "grad_out")
    _check_input(w12_out, "w12_out")
    if w12_out.dim() != 2 or w12_out.shape[1] != 2 * hidden_dim:
        raise RuntimeError("w12_out must be [M, 2*hidden_dim]")
    m = w12_out.shape[0]
    if tuple(grad_out.shape) != (m, hidden_dim):
        raise RuntimeError("grad_out must be [M, hidden_dim]")
    if grad_out.dtype != w12_out.dtype or grad_out.device != w12_out.device:
        raise RuntimeError("grad_out and w12_out must share dtype and device")
    code = _dtype_code(w12_out, " for backward")
    L = _capi.lib()
    with torch.cuda.device(w12_out.device):
        grad_in = torch.empty_like(w12_out)
        st = L.mgr_swiglu_act_bwd(grad_in.data_ptr(), grad_out.data_ptr(), w12_out.data_ptr(), m, hidden_dim, code,
                                  _stream_ptr(w12_out.device))
    _capi.check("SwiGLU activation backward kernel", st)
    return grad_in


def _gemm_ok(*tensors: torch.Tensor) -> bool:
    """True when the tensor-core kernels can take these operands: CUDA, fp16/bf16, contiguous 2-D with
    every dimension a multiple of 8 and 16-byte aligned storage."""
    dt = tensors[0].dtype
    if dt not in (torch.float16, torch.bfloat16):
        return False
    for t in tensors:
        if not (t.is_cuda and t.dtype == dt and t.dim() == 2 and t.is_contiguous() and t.data_ptr() % 16 == 0):
            return False
        if t.shape[0] < 0 or t.shape[1] % 8 != 0:
            return False
    return True


def swiglu_fused_forward(x: torch.Tensor, w12: torch.Tensor, hidden_dim: int, out: torch.Tensor | None = None,
                         row_scale: torch.Tensor | None = None) -> torch.Tensor:
    """h[M, hidden] = silu(x w12[:hidden]^T) * (x w12[hidden:]^T) in one tensor-core kernel: what
    `self.w12(x)` followed by MegaGemmFunction computes (megagemm/swiglu.py:167-168), without the
    [M, 2*hidden] intermediate. `row_scale` [M] fp32, if given, multiplies both halves of row r before the
    activation (an RMSNorm in front whose weight has been folded into w12: see swiglu.PreNormSwiGLU)."""
    _check_input(x, "x")
    _check_input(w12, "w12")
    if row_scale is not None:
        _check_input(row_scale, "row_scale")
        if row_scale.dtype != torch.float32 or tuple(row_scale.shape) != (x.shape[0],) or row_scale.device != x.device:
            raise RuntimeError("row_scale must be a float32 tensor [M] on the operands' device")
    if x.dim() != 2 or w12.dim() != 2 or w12.shape[0] != 2 * hidden_dim or w12.shape[1] != x.shape[1]:
        raise RuntimeError("expected x [M, d_model] and w12 [2*hidden_dim, d_model]")
    if x.dtype != w12.dtype or x.device != w12.device:
        raise RuntimeError("x and w12 must share dtype and device")
    code = _dtype_code(x, "")
    m, d = x.shape
    L = _capi.lib()
    with torch.cuda.device(x.device):
        h = _out_or_new(out, (m, hidden_dim), x, "out")
        st = L.mgr_swiglu_fused_fwd_scaled(h.data_ptr(), x.data_ptr(), w12.data_ptr(),
                                           row_scale.data_ptr() if row_scale is not None else None, m, d, hidden_dim, code,
                                           _stream_ptr(x.device))
    _capi.check("fused SwiGLU projection kernel", st)
    return h


def linear_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a [M, K] x b [N, K]^T -> [M, N] on the tensor-core kernel (an nn.Linear without bias). `out`, if
    given, is a contiguous [M, N] tensor to write into (e.g. a row slab of a larger result)."""
    _check_input(a, "a")
    _check_input(b, "b")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise RuntimeError("expected a [M, K] and b [N, K]")
    if a.dtype != b.dtype or a.device != b.device:
        raise RuntimeError("a and b must share dtype and device")
    code = _dtype_code(a, "")
    m, k = a.shape
    n = b.shape[0]
    L = _capi.lib()
    with torch.cuda.device(a.device):
        if out is None:
            c = torch.empty((m, n), device=a.device, dtype=a.dtype)
        else:
            if tuple(out.shape) != (m, n) or out.dtype != a.dtype or out.device != a.device or not out.is_contiguous():
                raise RuntimeError("out must be a contiguous [M, N] tensor of the operands' dtype and device")
            c = out
        st = L.mgr_gemm_tn(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, k, k, n, code, _stream_ptr(a.device))
    _capi.check("tensor-core GEMM kernel", st)
    return c


def gemm(a: torch.Tensor, b: torch.Tensor, a_mn_major: bool = False, b_mn_major: bool = False,
         out: torch.Tensor | None = None) -> torch.Tensor:
    """c[m, n] = op(a) op(b)^T on the tensor-core kernel. K-major operands are stored [m, k] / [n, k];
    MN-major ones are stored [k, m] / [k, n] (the transposed matrix as it already lies in memory), so
    the backward GEMMs of an nn.Linear need no transposed copy."""
    _check_input(a, "a")
    _check_input(b, "b")
    if a.dim() != 2 or b.dim() != 2:
        raise RuntimeError("operands must be 2-D")
    k, m = (a.shape if a_mn_major else a.shape[::-1])
    kb, n = (b.shape if b_mn_major else b.shape[::-1])
    if k != kb:
        raise RuntimeError("contraction lengths differ")
    if a.dtype != b.dtype or a.device != b.device:
        raise RuntimeError("operands must share dtype and device")
    code = _dtype_code(a, "")
    L = _capi.lib()
    with torch.cuda.device(a.device):
        c = _out_or_new(out, (m, n), a, "out")
        st = L.mgr_gemm(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, a.shape[1], b.shape[1], n,
                        int(a_mn_major), int(b_mn_major), code, _stream_ptr(a.device))
    _capi.check("tensor-core GEMM kernel", st)
    return c


def swiglu_fused_backward(dh: torch.Tensor, x: torch.Tensor, w12: torch.Tensor, hidden_dim: int) -> torch.Tensor:
    """[d_gate | d_val] of shape [M, 2*hidden] from dh [M, hidden], recomputing x w12^T inside the kernel
    (the recomputed `self.w12(x)` plus the launch at megagemm/swiglu.py:125-129, fused)."""
    for t, nme in ((dh, "dh"), (x, "x"), (w12, "w12")):
        _check_input(t, nme)
    m, d = x.shape
    if tuple(dh.shape) != (m, hidden_dim) or tuple(w12.shape) != (2 * hidden_dim, d):
        raise RuntimeError("expected dh [M, hidden], x [M, d_model], w12 [2*hidden, d_model]")
    if not (dh.dtype == x.dtype == w12.dtype) or not (dh.device == x.device == w12.device):
        raise RuntimeError("dh, x and w12 must share dtype and device")
    code = _dtype_code(x, " for backward")
    L = _capi.lib()
    with torch.cuda.device(x.device):
        dgv = torch.empty((m, 2 * hidden_dim), device=x.device, dtype=x.dtype)
        st = L.mgr_swiglu_fused_bwd(dgv.data_ptr(), dh.data_ptr(), x.data_ptr(), w12.data_ptr(), m, d, hidden_dim, code,
                                    _stream_ptr(x.device))
    _capi.check("fused SwiGLU backward kernel", st)
    return dgv


def swiglu_fused_forward_save(x: torch.Tensor, w12: torch.Tensor, hidden_dim: int, out_h: torch.Tensor | None = None,
                              out_gv: torch.Tensor | None = None):
    """(h[M, hidden], gv[M, 2*hidden]): the fused projection that also keeps the projection for backward,
    as the reference keeps w12_out (megagemm/swiglu.py:98)."""
    _check_input(x, "x")
    _check_input(w12, "w12")
    if x.dim() != 2 or w12.dim() != 2 or w12.shape[0] != 2 * hidden_dim or w12.shape[1] != x.shape[1]:
        raise RuntimeError("expected x [M, d_model] and w12 [2*hidden_dim, d_model]")
    if x.dtype != w12.dtype or x.device != w12.device:
        raise RuntimeError("x and w12 must share dtype and device")
    code = _dtype_code(x, "")
    m, d = x.shape
    L = _capi.lib()
    with torch.cuda.device(x.device):
        h = _out_or_new(out_h, (m, hidden_dim), x, "out_h")
        gv = _out_or_new(out_gv, (m, 2 * hidden_dim), x, "out_gv")
        st = L.mgr_swiglu_fused_fwd_save(h.data_ptr(), gv.data_ptr(), x.data_ptr(), w12.data_ptr(), m, d, hidden_dim, code,
                                         _stream_ptr(x.device))
    _capi.check("fused SwiGLU projection kernel", st)
    return h, gv


def swiglu_dh_dgv(dy: torch.Tensor, w3: torch.Tensor, gv: torch.Tensor, hidden_dim: int,
                  out: torch.Tensor | None = None) -> torch.Tensor:
    """[d_gate | d_val] of shape [M, 2*hidden] from dy [M, d_model], w3 [d_model, hidden] and the stored
    projection gv: the dh = dy w3 GEMM with the activation backward as its epilogue."""
    for t, nme in ((dy, "dy"), (w3, "w3"), (gv, "gv")):
        _check_input(t, nme)
    m, d = dy.shape
    if tuple(w3.shape) != (d, hidden_dim) or tuple(gv.shape) != (m, 2 * hidden_dim):
        raise RuntimeError("expected dy [M, d_model], w3 [d_model, hidden], gv [M, 2*hidden]")
    if not (dy.dtype == w3.dtype == gv.dtype) or not (dy.device == w3.device == gv.device):
        raise RuntimeError("dy, w3 and gv must share dtype and device")
    code = _dtype_code(dy, " for backward")
    L = _capi.lib()
    with torch.cuda.device(dy.device):
        dgv = _out_or_new(out, gv.shape, gv, "out")
        st = L.mgr_swiglu_dh_dgv(dgv.data_ptr(), dy.data_ptr(), w3.data_ptr(), gv.data_ptr(), m, d, hidden_dim, code,
                                 _stream_ptr(dy.device))
    _capi.check("fused dh/dGV kernel", st)
    return dgv


class gemm_sm_limit:
    """Context manager: leaves `reserve` SMs free of GEMM CTAs while it is active (for a collective that
    runs beside the GEMMs launched inside it)."""

    def __init__(self, reserve: int, device=None):
        self.reserve = reserve
        self.device = device

    def __enter__(self):
        sms = torch.cuda.get_device_properties(self.device if self.device is not None else torch.cuda.current_device()).multi_processor_count
        self.prev = _capi.lib().mgr_gemm_set_sm_limit(max(2, sms - self.reserve) if self.reserve > 0 else 0)
        return self

    def __exit__(self, *exc):
        _capi.lib().mgr_gemm_set_sm_limit(self.prev)
        return False


def device_status(clear: bool = True) -> None:
    """Raises if a kernel on the current device gave up a bounded wait since the last clearing read
    (mgr_device_status). Outputs of such a launch are incomplete. This call synchronises with the device, so
    it belongs where the host waits anyway: after a step's final synchronisation, before results are used."""
    _capi.check("device status", _capi.lib().mgr_device_status(1 if clear else 0))


# ---------------------------------------------------------------------------------------------------
# route selection
# ---------------------------------------------------------------------------------------------------

ENTRY_POINTS = ("rmsnorm_forward", "rms_inv", "rmsnorm_backward", "rmsnorm_backward_full", "add_rmsnorm_forward", "add_rmsnorm_backward",
                "swiglu_act_forward", "swiglu_act_backward", "swiglu_fused_forward", "swiglu_fused_forward_save", "linear_tn",
                "gemm", "swiglu_fused_backward", "swiglu_dh_dgv")
ctypes_impl = {name: globals()[name] for name in ENTRY_POINTS}


def _compiled_binding():
    if os.environ.get("MGR_BINDING", "") == "ctypes":
        return None
    try:
        _capi.lib()                      # the extension links against the library: load it (or fail loudly) first
        from .pybind import rmsnorm_cuda_ops as ext
    except ImportError:
        return None
    return ext


compiled = _compiled_binding()
BINDING = "ctypes" if compiled is None else "pybind"
if compiled is not None:
    for _name in ENTRY_POINTS:
        globals()[_name] = getattr(compiled, _name)
