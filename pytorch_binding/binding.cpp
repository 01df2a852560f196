// `rmsnorm_cuda_ops` as a compiled torch extension over the C ABI of libmgr_b200.so.
//
// Takes the place of the reference's pytorch_binding/binding.cpp: the same two Python-visible functions
// (rmsnorm_forward / rmsnorm_backward, binding.cpp:136-139) with the same duties -- check the tensors
// (:9-11, :17-24, :79-82), allocate the outputs through torch (:29-30, :89-90), dispatch on the input
// dtype (:34-63, :94-129), raise RuntimeError on failure (:65, :131) -- but the calls go to
// include/mgr_b200.h instead of src/rmsnorm_kernel.h. Two things the reference's binding lacks are added:
// a device guard, and launches on torch's current stream (the reference launches on the legacy default
// stream of whichever device happens to be current, src/rmsnorm_kernel.cu:542,564).
//
// The SwiGLU entry points below have no counterpart in the reference's binding (its activation is a
// Triton kernel inside megagemm/swiglu.py:18-79 and its GEMMs are nn.Linear); they are what
// mgrrmsnorm_b200/swiglu.py calls instead.
//
// No arithmetic happens here and no torch kernel is launched: torch supplies memory and the stream.

#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

#include <algorithm>
#include <optional>
#include <vector>

#include "mgr_b200.h"

namespace {

using at::Tensor;

void check_input(const Tensor& t, const char* name) {
    TORCH_CHECK(t.device().is_cuda(), name, " must be a CUDA tensor");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

int dtype_code(const Tensor& t, const char* what) {
    switch (t.scalar_type()) {
        case at::kFloat: return MGR_F32;
        case at::kHalf: return MGR_F16;
        case at::kBFloat16: return MGR_BF16;
        default: TORCH_CHECK(false, "Unsupported dtype", what, ". Use float32, float16, or bfloat16.");
    }
    return -1;
}

void check_status(const char* what, int st) {
    TORCH_CHECK(st == MGR_OK, what, " failed: ", mgr_status_str(st), " (status ", st, ")");
}

void* current_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

Tensor out_or_new(const std::optional<Tensor>& out, at::IntArrayRef shape, const Tensor& like, const char* name) {
    if (!out.has_value()) return at::empty(shape, like.options());
    const Tensor& o = *out;
    TORCH_CHECK(o.sizes() == shape && o.scalar_type() == like.scalar_type() && o.device() == like.device() && o.is_contiguous(),
                name, " must be a contiguous ", shape, " tensor of the operands' dtype and device");
    return o;
}

Tensor workspace_for(int64_t rows, int64_t cols, int code, const Tensor& like) {
    const size_t need = mgr_rmsnorm_bwd_workspace_bytes(rows, cols, code);
    return at::empty({static_cast<int64_t>(std::max<size_t>(need, 16))}, like.options().dtype(at::kByte));
}

// ---- RMSNorm ----------------------------------------------------------------------------------------

std::vector<Tensor> rmsnorm_forward(const Tensor& input, const Tensor& weight, double epsilon) {
    check_input(input, "input");
    check_input(weight, "weight");
    TORCH_CHECK(input.dim() == 2, "Input must be 2D");
    const int64_t rows = input.size(0), cols = input.size(1);
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == cols, "Weight size must match hidden size");
    const int code = dtype_code(input, "");
    TORCH_CHECK(weight.scalar_type() == input.scalar_type(), "weight dtype ", weight.scalar_type(), " must match input dtype ",
                input.scalar_type());
    TORCH_CHECK(weight.device() == input.device(), "input and weight must be on the same device");
    c10::cuda::CUDAGuard guard(input.device());
    Tensor inv_rms = at::empty({rows}, input.options().dtype(at::kFloat));
    Tensor output = at::empty_like(input);
    const int st = mgr_rmsnorm_fwd(output.data_ptr(), inv_rms.data_ptr<float>(), input.data_ptr(), weight.data_ptr(), rows, cols,
                                   static_cast<float>(epsilon), code, current_stream());
    check_status("RMSNorm Forward CUDA kernel", st);
    return {output, inv_rms};
}

// The forward's row scales alone (one read of the input); same bits as the inv_rms rmsnorm_forward returns.
Tensor rms_inv(const Tensor& input, double epsilon) {
    check_input(input, "input");
    TORCH_CHECK(input.dim() == 2, "Input must be 2D");
    const int code = dtype_code(input, "");
    c10::cuda::CUDAGuard guard(input.device());
    Tensor inv_rms = at::empty({input.size(0)}, input.options().dtype(at::kFloat));
    check_status("RMSNorm row-scale CUDA kernel", mgr_rms_inv(inv_rms.data_ptr<float>(), input.data_ptr(), input.size(0), input.size(1),
                                                            static_cast<float>(epsilon), code, current_stream()));
    return inv_rms;
}

// [grad_input, grad_weight, grad_weight_fp32 or None]; the fp32 sum is what a row-sharded caller all-reduces
// across ranks before the one rounding.
std::vector<std::optional<Tensor>> rmsnorm_backward_full(const Tensor& grad_output, const Tensor& input, const Tensor& weight,
                                                         const Tensor& inv_rms, bool want_dw_f32) {
    check_input(grad_output, "grad_output");
    check_input(input, "input");
    check_input(weight, "weight");
    check_input(inv_rms, "inv_rms");
    TORCH_CHECK(input.dim() == 2, "Input must be 2D");
    const int64_t rows = input.size(0), cols = input.size(1);
    TORCH_CHECK(grad_output.sizes() == input.sizes(), "grad_output shape must match input shape");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == cols, "Weight size must match hidden size");
    TORCH_CHECK(inv_rms.scalar_type() == at::kFloat && inv_rms.numel() == rows, "inv_rms must be a float32 tensor with one value per row");
    const int code = dtype_code(input, " for backward");
    TORCH_CHECK(grad_output.scalar_type() == input.scalar_type() && weight.scalar_type() == input.scalar_type(),
                "grad_output, input and weight must share one dtype");
    TORCH_CHECK(grad_output.device() == input.device() && weight.device() == input.device() && inv_rms.device() == input.device(),
                "all tensors must be on the same device");
    c10::cuda::CUDAGuard guard(input.device());
    Tensor grad_input = at::empty_like(input);
    Tensor grad_weight = at::empty_like(weight);   // fully overwritten by the library: no memset (reference: :562)
    std::optional<Tensor> dw_f32;
    if (want_dw_f32) dw_f32 = at::empty({cols}, input.options().dtype(at::kFloat));
    Tensor ws = workspace_for(rows, cols, code, input);
    const int st = mgr_rmsnorm_bwd(grad_input.data_ptr(), grad_weight.data_ptr(), dw_f32 ? dw_f32->data_ptr<float>() : nullptr,
                                   grad_output.data_ptr(), input.data_ptr(), weight.data_ptr(), inv_rms.data_ptr<float>(), rows, cols,
                                   code, ws.data_ptr(), static_cast<size_t>(ws.numel()), current_stream());
    check_status("RMSNorm Backward CUDA kernel", st);
    return {grad_input, grad_weight, dw_f32};
}

std::vector<Tensor> rmsnorm_backward(const Tensor& grad_output, const Tensor& input, const Tensor& weight, const Tensor& inv_rms) {
    auto r = rmsnorm_backward_full(grad_output, input, weight, inv_rms, false);
    return {*r[0], *r[1]};
}

std::vector<Tensor> add_rmsnorm_forward(const Tensor& input, const Tensor& residual, const Tensor& weight, double epsilon, bool inplace) {
    check_input(input, "input");
    check_input(residual, "residual");
    check_input(weight, "weight");
    TORCH_CHECK(input.dim() == 2, "Input must be 2D");
    const int64_t rows = input.size(0), cols = input.size(1);
    TORCH_CHECK(residual.sizes() == input.sizes(), "residual shape must match input shape");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == cols, "Weight size must match hidden size");
    const int code = dtype_code(input, "");
    TORCH_CHECK(weight.scalar_type() == input.scalar_type() && residual.scalar_type() == input.scalar_type(),
                "input, residual and weight must share one dtype");
    TORCH_CHECK(residual.device() == input.device() && weight.device() == input.device(), "all tensors must be on the same device");
    c10::cuda::CUDAGuard guard(input.device());
    Tensor inv_rms = at::empty({rows}, input.options().dtype(at::kFloat));
    Tensor output = at::empty_like(input);
    Tensor hidden = inplace ? residual : at::empty_like(input);
    const int st = mgr_add_rmsnorm_fwd(output.data_ptr(), hidden.data_ptr(), inv_rms.data_ptr<float>(), input.data_ptr(),
                                       residual.data_ptr(), weight.data_ptr(), rows, cols, static_cast<float>(epsilon), code,
                                       current_stream());
    check_status("Add+RMSNorm Forward CUDA kernel", st);
    return {output, hidden, inv_rms};
}

std::vector<std::optional<Tensor>> add_rmsnorm_backward(const Tensor& grad_output, const Tensor& grad_hidden, const Tensor& hidden,
                                                        const Tensor& weight, const Tensor& inv_rms, bool want_dw_f32) {
    check_input(grad_output, "grad_output");
    check_input(grad_hidden, "grad_hidden");
    check_input(hidden, "hidden");
    check_input(weight, "weight");
    check_input(inv_rms, "inv_rms");
    TORCH_CHECK(hidden.dim() == 2, "Input must be 2D");
    const int64_t rows = hidden.size(0), cols = hidden.size(1);
    TORCH_CHECK(grad_output.sizes() == hidden.sizes() && grad_hidden.sizes() == hidden.sizes(), "gradient shapes must match the hidden shape");
    TORCH_CHECK(weight.dim() == 1 && weight.size(0) == cols, "Weight size must match hidden size");
    TORCH_CHECK(inv_rms.scalar_type() == at::kFloat && inv_rms.numel() == rows, "inv_rms must be a float32 tensor with one value per row");
    const int code = dtype_code(hidden, " for backward");
    TORCH_CHECK(grad_output.scalar_type() == hidden.scalar_type() && grad_hidden.scalar_type() == hidden.scalar_type() &&
                    weight.scalar_type() == hidden.scalar_type(),
                "grad_output, grad_hidden, hidden and weight must share one dtype");
    TORCH_CHECK(grad_output.device() == hidden.device() && grad_hidden.device() == hidden.device() &&
                    weight.device() == hidden.device() && inv_rms.device() == hidden.device(),
                "all tensors must be on the same device");
    c10::cuda::CUDAGuard guard(hidden.device());
    Tensor grad_total = at::empty_like(hidden);
    Tensor grad_weight = at::empty_like(weight);
    std::optional<Tensor> dw_f32;
    if (want_dw_f32) dw_f32 = at::empty({cols}, hidden.options().dtype(at::kFloat));
    Tensor ws = workspace_for(rows, cols, code, hidden);
    const int st = mgr_add_rmsnorm_bwd(grad_total.data_ptr(), grad_weight.data_ptr(), dw_f32 ? dw_f32->data_ptr<float>() : nullptr,
                                       grad_output.data_ptr(), grad_hidden.data_ptr(), hidden.data_ptr(), weight.data_ptr(),
                                       inv_rms.data_ptr<float>(), rows, cols, code, ws.data_ptr(), static_cast<size_t>(ws.numel()),
                                       current_stream());
    check_status("Add+RMSNorm Backward CUDA kernel", st);
    return {grad_total, grad_weight, dw_f32};
}

// ---- SwiGLU -----------------------------------------------------------------------------------------

Tensor swiglu_act_forward(const Tensor& w12_out, int64_t hidden_dim) {
    check_input(w12_out, "w12_out");
    TORCH_CHECK(w12_out.dim() == 2 && w12_out.size(1) == 2 * hidden_dim, "w12_out must be [M, 2*hidden_dim]");
    const int code = dtype_code(w12_out, "");
    const int64_t m = w12_out.size(0);
    c10::cuda::CUDAGuard guard(w12_out.device());
    Tensor out = at::empty({m, hidden_dim}, w12_out.options());
    check_status("SwiGLU activation forward kernel",
                 mgr_swiglu_act_fwd(out.data_ptr(), w12_out.data_ptr(), m, hidden_dim, code, current_stream()));
    return out;
}

Tensor swiglu_act_backward(const Tensor& grad_out, const Tensor& w12_out, int64_t hidden_dim) {
    check_input(grad_out, "grad_out");
    check_input(w12_out, "w12_out");
    TORCH_CHECK(w12_out.dim() == 2 && w12_out.size(1) == 2 * hidden_dim, "w12_out must be [M, 2*hidden_dim]");
    const int64_t m = w12_out.size(0);
    TORCH_CHECK(grad_out.dim() == 2 && grad_out.size(0) == m && grad_out.size(1) == hidden_dim, "grad_out must be [M, hidden_dim]");
    TORCH_CHECK(grad_out.scalar_type() == w12_out.scalar_type() && grad_out.device() == w12_out.device(),
                "grad_out and w12_out must share dtype and device");
    const int code = dtype_code(w12_out, " for backward");
    c10::cuda::CUDAGuard guard(w12_out.device());
    Tensor grad_in = at::empty_like(w12_out);
    check_status("SwiGLU activation backward kernel",
                 mgr_swiglu_act_bwd(grad_in.data_ptr(), grad_out.data_ptr(), w12_out.data_ptr(), m, hidden_dim, code, current_stream()));
    return grad_in;
}

void check_projection_operands(const Tensor& x, const Tensor& w12, int64_t hidden_dim) {
    check_input(x, "x");
    check_input(w12, "w12");
    TORCH_CHECK(x.dim() == 2 && w12.dim() == 2 && w12.size(0) == 2 * hidden_dim && w12.size(1) == x.size(1),
                "expected x [M, d_model] and w12 [2*hidden_dim, d_model]");
    TORCH_CHECK(x.scalar_type() == w12.scalar_type() && x.device() == w12.device(), "x and w12 must share dtype and device");
}

Tensor swiglu_fused_forward(const Tensor& x, const Tensor& w12, int64_t hidden_dim, const std::optional<Tensor>& out,
                            const std::optional<Tensor>& row_scale) {
    check_projection_operands(x, w12, hidden_dim);
    const int code = dtype_code(x, "");
    const int64_t m = x.size(0), d = x.size(1);
    const float* scale = nullptr;
    if (row_scale.has_value()) {
        check_input(*row_scale, "row_scale");
        TORCH_CHECK(row_scale->scalar_type() == at::kFloat && row_scale->dim() == 1 && row_scale->size(0) == m &&
                        row_scale->device() == x.device(),
                    "row_scale must be a float32 tensor [M] on the operands' device");
        scale = row_scale->data_ptr<float>();
    }
    c10::cuda::CUDAGuard guard(x.device());
    Tensor h = out_or_new(out, {m, hidden_dim}, x, "out");
    check_status("fused SwiGLU projection kernel",
                 mgr_swiglu_fused_fwd_scaled(h.data_ptr(), x.data_ptr(), w12.data_ptr(), scale, m, d, hidden_dim, code, current_stream()));
    return h;
}

std::vector<Tensor> swiglu_fused_forward_save(const Tensor& x, const Tensor& w12, int64_t hidden_dim, const std::optional<Tensor>& out_h,
                                              const std::optional<Tensor>& out_gv) {
    check_projection_operands(x, w12, hidden_dim);
    const int code = dtype_code(x, "");
    const int64_t m = x.size(0), d = x.size(1);
    c10::cuda::CUDAGuard guard(x.device());
    Tensor h = out_or_new(out_h, {m, hidden_dim}, x, "out_h");
    Tensor gv = out_or_new(out_gv, {m, 2 * hidden_dim}, x, "out_gv");
    check_status("fused SwiGLU projection kernel",
                 mgr_swiglu_fused_fwd_save(h.data_ptr(), gv.data_ptr(), x.data_ptr(), w12.data_ptr(), m, d, hidden_dim, code, current_stream()));
    return {h, gv};
}

Tensor gemm(const Tensor& a, const Tensor& b, bool a_mn_major, bool b_mn_major, const std::optional<Tensor>& out) {
    check_input(a, "a");
    check_input(b, "b");
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "operands must be 2-D");
    const int64_t k = a_mn_major ? a.size(0) : a.size(1), m = a_mn_major ? a.size(1) : a.size(0);
    const int64_t kb = b_mn_major ? b.size(0) : b.size(1), n = b_mn_major ? b.size(1) : b.size(0);
    TORCH_CHECK(k == kb, "contraction lengths differ");
    TORCH_CHECK(a.scalar_type() == b.scalar_type() && a.device() == b.device(), "operands must share dtype and device");
    const int code = dtype_code(a, "");
    c10::cuda::CUDAGuard guard(a.device());
    Tensor c = out_or_new(out, {m, n}, a, "out");
    check_status("tensor-core GEMM kernel", mgr_gemm(c.data_ptr(), a.data_ptr(), b.data_ptr(), m, n, k, a.size(1), b.size(1), n,
                                                     a_mn_major ? 1 : 0, b_mn_major ? 1 : 0, code, current_stream()));
    return c;
}

Tensor linear_tn(const Tensor& a, const Tensor& b, const std::optional<Tensor>& out) {
    TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && a.size(1) == b.size(1), "expected a [M, K] and b [N, K]");
    return gemm(a, b, false, false, out);
}

Tensor swiglu_fused_backward(const Tensor& dh, const Tensor& x, const Tensor& w12, int64_t hidden_dim) {
    check_input(dh, "dh");
    check_input(x, "x");
    check_input(w12, "w12");
    TORCH_CHECK(x.dim() == 2, "expected dh [M, hidden], x [M, d_model], w12 [2*hidden, d_model]");
    const int64_t m = x.size(0), d = x.size(1);
    TORCH_CHECK(dh.dim() == 2 && dh.size(0) == m && dh.size(1) == hidden_dim && w12.dim() == 2 && w12.size(0) == 2 * hidden_dim &&
                    w12.size(1) == d,
                "expected dh [M, hidden], x [M, d_model], w12 [2*hidden, d_model]");
    TORCH_CHECK(dh.scalar_type() == x.scalar_type() && w12.scalar_type() == x.scalar_type() && dh.device() == x.device() &&
                    w12.device() == x.device(),
                "dh, x and w12 must share dtype and device");
    const int code = dtype_code(x, " for backward");
    c10::cuda::CUDAGuard guard(x.device());
    Tensor dgv = at::empty({m, 2 * hidden_dim}, x.options());
    check_status("fused SwiGLU backward kernel",
                 mgr_swiglu_fused_bwd(dgv.data_ptr(), dh.data_ptr(), x.data_ptr(), w12.data_ptr(), m, d, hidden_dim, code, current_stream()));
    return dgv;
}

Tensor swiglu_dh_dgv(const Tensor& dy, const Tensor& w3, const Tensor& gv, int64_t hidden_dim, const std::optional<Tensor>& out) {
    check_input(dy, "dy");
    check_input(w3, "w3");
    check_input(gv, "gv");
    TORCH_CHECK(dy.dim() == 2, "expected dy [M, d_model], w3 [d_model, hidden], gv [M, 2*hidden]");
    const int64_t m = dy.size(0), d = dy.size(1);
    TORCH_CHECK(w3.dim() == 2 && w3.size(0) == d && w3.size(1) == hidden_dim && gv.dim() == 2 && gv.size(0) == m &&
                    gv.size(1) == 2 * hidden_dim,
                "expected dy [M, d_model], w3 [d_model, hidden], gv [M, 2*hidden]");
    TORCH_CHECK(dy.scalar_type() == w3.scalar_type() && gv.scalar_type() == dy.scalar_type() && dy.device() == w3.device() &&
                    gv.device() == dy.device(),
                "dy, w3 and gv must share dtype and device");
    const int code = dtype_code(dy, " for backward");
    c10::cuda::CUDAGuard guard(dy.device());
    Tensor dgv = out_or_new(out, gv.sizes(), gv, "out");
    check_status("fused dh/dGV kernel",
                 mgr_swiglu_dh_dgv(dgv.data_ptr(), dy.data_ptr(), w3.data_ptr(), gv.data_ptr(), m, d, hidden_dim, code, current_stream()));
    return dgv;
}

int64_t device_status(bool clear) { return mgr_device_status(clear ? 1 : 0); }
int64_t set_gemm_sm_limit(int64_t sms) { return mgr_gemm_set_sm_limit(static_cast<int>(sms)); }

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "rmsnorm_cuda_ops: torch binding of libmgr_b200.so (sm_100a RMSNorm and SwiGLU kernels)";
    m.def("rmsnorm_forward", &rmsnorm_forward, "RMSNorm forward (CUDA): [output, inv_rms]", py::arg("input"), py::arg("weight"),
          py::arg("epsilon"));
    m.def("rmsnorm_backward", &rmsnorm_backward, "RMSNorm backward (CUDA): [grad_input, grad_weight]", py::arg("grad_output"),
          py::arg("input"), py::arg("weight"), py::arg("inv_rms"));
    m.def("rmsnorm_backward_full", &rmsnorm_backward_full, "[grad_input, grad_weight, grad_weight_fp32 | None]", py::arg("grad_output"),
          py::arg("input"), py::arg("weight"), py::arg("inv_rms"), py::arg("want_dw_f32") = false);
    m.def("add_rmsnorm_forward", &add_rmsnorm_forward, "[output, hidden, inv_rms] of RMSNorm(input + residual)", py::arg("input"),
          py::arg("residual"), py::arg("weight"), py::arg("epsilon"), py::arg("inplace") = false);
    m.def("add_rmsnorm_backward", &add_rmsnorm_backward, "[grad_hidden_total, grad_weight, grad_weight_fp32 | None]",
          py::arg("grad_output"), py::arg("grad_hidden"), py::arg("hidden"), py::arg("weight"), py::arg("inv_rms"),
          py::arg("want_dw_f32") = false);
    m.def("swiglu_act_forward", &swiglu_act_forward, py::arg("w12_out"), py::arg("hidden_dim"));
    m.def("swiglu_act_backward", &swiglu_act_backward, py::arg("grad_out"), py::arg("w12_out"), py::arg("hidden_dim"));
    m.def("swiglu_fused_forward", &swiglu_fused_forward, py::arg("x"), py::arg("w12"), py::arg("hidden_dim"), py::arg("out") = py::none(),
          py::arg("row_scale") = py::none());
    m.def("rms_inv", &rms_inv, "inv_rms [rows] fp32 of a 2-D tensor (the forward's row scales alone)", py::arg("input"), py::arg("epsilon"));
    m.def("swiglu_fused_forward_save", &swiglu_fused_forward_save, py::arg("x"), py::arg("w12"), py::arg("hidden_dim"),
          py::arg("out_h") = py::none(), py::arg("out_gv") = py::none());
    m.def("linear_tn", &linear_tn, py::arg("a"), py::arg("b"), py::arg("out") = py::none());
    m.def("gemm", &gemm, py::arg("a"), py::arg("b"), py::arg("a_mn_major") = false, py::arg("b_mn_major") = false,
          py::arg("out") = py::none());
    m.def("swiglu_fused_backward", &swiglu_fused_backward, py::arg("dh"), py::arg("x"), py::arg("w12"), py::arg("hidden_dim"));
    m.def("swiglu_dh_dgv", &swiglu_dh_dgv, py::arg("dy"), py::arg("w3"), py::arg("gv"), py::arg("hidden_dim"), py::arg("out") = py::none());
    m.def("device_status", &device_status, "mgr_device_status(clear)", py::arg("clear") = true);
    m.def("set_gemm_sm_limit", &set_gemm_sm_limit, "mgr_gemm_set_sm_limit(sms): returns the previous limit", py::arg("sms"));
}
