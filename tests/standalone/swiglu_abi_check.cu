// Torch-free check of the MLP half of the C ABI: a plain C++ host program that links libmgr_b200.so and
// runs one SwiGLU MLP forward + backward through the entry points a binding would call, in the order
// megagemm/swiglu.py:163-169 and its autograd imply:
//   forward : mgr_swiglu_fused_fwd_save (x w12^T -> h, [gate|val])      mgr_gemm_tn (y = h w3^T)
//   backward: mgr_gemm (dW3 = dy^T h)   mgr_swiglu_dh_dgv (dy w3 -> [d_gate|d_val])
//             mgr_gemm (dx = dGV w12)   mgr_gemm (dW12 = dGV^T x)
// fp16, 200 tokens, d_model 256, hidden 384, weights U(-1/sqrt(fan_in), 1/sqrt(fan_in)) as nn.Linear draws
// them. Every result is compared with the CPU oracle (mgr_oracle.c, linked in) evaluated in fp64 on the same
// fp16 inputs; the bound is the one the reference's benchmark applies to its forward, 1e-2
// (benchmark_swiglu.py:121-129), scaled by the magnitude of the weight gradients. Prints one line per check
// and exits non-zero on failure.
//
// Build (from the repository root):
//   nvcc -O2 -std=c++17 -Iinclude tests/standalone/swiglu_abi_check.cu oracle/mgr_oracle.c \
//        -Lmgrrmsnorm_b200/lib -lmgr_b200 -Xlinker -rpath=$PWD/mgrrmsnorm_b200/lib -o /tmp/swiglu_abi_check
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <random>
#include <vector>

#include "mgr_b200.h"

extern "C" {
void mgr_oracle_swiglu_act_fwd_f64(double* h, const float* gv, int64_t m, int64_t f);
void mgr_oracle_swiglu_act_bwd_f64(double* dgv, const float* dh, const float* gv, int64_t m, int64_t f);
void mgr_oracle_linear_f64(double* c, const float* a, const float* b, int64_t m, int64_t n, int64_t k);
}

#define CUDA_OK(call)                                                                        \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess) {                                                             \
            std::fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_));          \
            return 2;                                                                        \
        }                                                                                    \
    } while (0)
#define MGR_OK_OR_DIE(call)                                                                  \
    do {                                                                                     \
        int s_ = (call);                                                                     \
        if (s_ != MGR_OK) {                                                                  \
            std::fprintf(stderr, "%s failed: %s\n", #call, mgr_status_str(s_));              \
            return 2;                                                                        \
        }                                                                                    \
    } while (0)

namespace {

// host copy of an fp16 matrix: the rounded values as float (what the oracle reads) and the raw halves (what the GPU reads)
struct HalfMat {
    std::vector<float> f;
    std::vector<__half> h;
    explicit HalfMat(size_t n) : f(n), h(n) {}
    void set(size_t i, float v) {
        h[i] = __float2half(v);
        f[i] = __half2float(h[i]);
    }
};

std::vector<float> transpose(const std::vector<float>& a, int64_t rows, int64_t cols) {
    std::vector<float> t(a.size());
    for (int64_t r = 0; r < rows; ++r)
        for (int64_t c = 0; c < cols; ++c) t[c * rows + r] = a[r * cols + c];
    return t;
}

std::vector<float> to_float(const std::vector<double>& d) { return std::vector<float>(d.begin(), d.end()); }

struct DevBuf {
    void* p = nullptr;
    ~DevBuf() { cudaFree(p); }
};

bool report(const char* what, const std::vector<__half>& got, const std::vector<double>& want, double rel) {
    double err = 0, scale = 0;
    for (size_t i = 0; i < got.size(); ++i) {
        err = std::fmax(err, std::fabs(static_cast<double>(__half2float(got[i])) - want[i]));
        scale = std::fmax(scale, std::fabs(want[i]));
    }
    const double bound = rel * std::fmax(1.0, scale);
    const bool ok = err <= bound;
    std::printf("%-6s max |err| %.3e (bound %.3e, max |truth| %.3g)  %s\n", what, err, bound, scale, ok ? "ok" : "FAILED");
    return ok;
}

}  // namespace

int main() {
    const int64_t M = 200, D = 256, F = 384;
    std::mt19937 gen(4321);
    std::normal_distribution<float> normal(0.0f, 1.0f);
    std::uniform_real_distribution<float> unit(-1.0f, 1.0f);

    HalfMat x(M * D), dy(M * D), w12(2 * F * D), w3(D * F);
    for (size_t i = 0; i < x.f.size(); ++i) x.set(i, normal(gen));
    for (size_t i = 0; i < dy.f.size(); ++i) dy.set(i, normal(gen));
    for (size_t i = 0; i < w12.f.size(); ++i) w12.set(i, unit(gen) / std::sqrt(static_cast<float>(D)));
    for (size_t i = 0; i < w3.f.size(); ++i) w3.set(i, unit(gen) / std::sqrt(static_cast<float>(F)));

    int sms = 0;
    MGR_OK_OR_DIE(mgr_device_check(&sms));
    std::printf("device: %d SMs, ABI version %d\n", sms, mgr_abi_version());

    // ---- fp64 truth on the CPU (oracle arithmetic on the fp16 inputs) ----
    std::vector<double> t_gv(M * 2 * F), t_h(M * F), t_y(M * D), t_dh(M * F), t_dgv(M * 2 * F), t_dx(M * D),
        t_dw3(D * F), t_dw12(2 * F * D);
    mgr_oracle_linear_f64(t_gv.data(), x.f.data(), w12.f.data(), M, 2 * F, D);
    const std::vector<float> gv_f = to_float(t_gv);
    mgr_oracle_swiglu_act_fwd_f64(t_h.data(), gv_f.data(), M, F);
    const std::vector<float> h_f = to_float(t_h);
    mgr_oracle_linear_f64(t_y.data(), h_f.data(), w3.f.data(), M, D, F);
    const std::vector<float> w3_t = transpose(w3.f, D, F);                 // [F, D]
    mgr_oracle_linear_f64(t_dh.data(), dy.f.data(), w3_t.data(), M, F, D);  // dh = dy w3
    const std::vector<float> dh_f = to_float(t_dh);
    mgr_oracle_swiglu_act_bwd_f64(t_dgv.data(), dh_f.data(), gv_f.data(), M, F);
    const std::vector<float> dgv_f = to_float(t_dgv);
    const std::vector<float> w12_t = transpose(w12.f, 2 * F, D);            // [D, 2F]
    mgr_oracle_linear_f64(t_dx.data(), dgv_f.data(), w12_t.data(), M, D, 2 * F);   // dx = dgv w12
    const std::vector<float> dy_t = transpose(dy.f, M, D), h_t = transpose(h_f, M, F);
    mgr_oracle_linear_f64(t_dw3.data(), dy_t.data(), h_t.data(), D, F, M);          // dW3 = dy^T h
    const std::vector<float> dgv_t = transpose(dgv_f, M, 2 * F), x_t = transpose(x.f, M, D);
    mgr_oracle_linear_f64(t_dw12.data(), dgv_t.data(), x_t.data(), 2 * F, D, M);    // dW12 = dgv^T x

    // ---- the same step on the GPU through the C ABI ----
    DevBuf d_x, d_dy, d_w12, d_w3, d_h, d_gv, d_y, d_dgv, d_dx, d_dw3, d_dw12;
    auto alloc = [](DevBuf& b, size_t halves) { return cudaMalloc(&b.p, halves * sizeof(__half)); };
    CUDA_OK(alloc(d_x, M * D));
    CUDA_OK(alloc(d_dy, M * D));
    CUDA_OK(alloc(d_w12, 2 * F * D));
    CUDA_OK(alloc(d_w3, D * F));
    CUDA_OK(alloc(d_h, M * F));
    CUDA_OK(alloc(d_gv, M * 2 * F));
    CUDA_OK(alloc(d_y, M * D));
    CUDA_OK(alloc(d_dgv, M * 2 * F));
    CUDA_OK(alloc(d_dx, M * D));
    CUDA_OK(alloc(d_dw3, D * F));
    CUDA_OK(alloc(d_dw12, 2 * F * D));
    CUDA_OK(cudaMemcpy(d_x.p, x.h.data(), x.h.size() * sizeof(__half), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_dy.p, dy.h.data(), dy.h.size() * sizeof(__half), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_w12.p, w12.h.data(), w12.h.size() * sizeof(__half), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_w3.p, w3.h.data(), w3.h.size() * sizeof(__half), cudaMemcpyHostToDevice));

    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    MGR_OK_OR_DIE(mgr_swiglu_fused_fwd_save(d_h.p, d_gv.p, d_x.p, d_w12.p, M, D, F, MGR_F16, stream));
    MGR_OK_OR_DIE(mgr_gemm_tn(d_y.p, d_h.p, d_w3.p, M, D, F, F, F, D, MGR_F16, stream));
    MGR_OK_OR_DIE(mgr_gemm(d_dw3.p, d_dy.p, d_h.p, D, F, M, D, F, F, 1, 1, MGR_F16, stream));
    MGR_OK_OR_DIE(mgr_swiglu_dh_dgv(d_dgv.p, d_dy.p, d_w3.p, d_gv.p, M, D, F, MGR_F16, stream));
    MGR_OK_OR_DIE(mgr_gemm(d_dx.p, d_dgv.p, d_w12.p, M, D, 2 * F, 2 * F, D, D, 0, 1, MGR_F16, stream));
    MGR_OK_OR_DIE(mgr_gemm(d_dw12.p, d_dgv.p, d_x.p, 2 * F, D, M, 2 * F, D, D, 1, 1, MGR_F16, stream));
    CUDA_OK(cudaStreamSynchronize(stream));
    MGR_OK_OR_DIE(mgr_device_status(1));

    auto fetch = [](const DevBuf& b, size_t n, std::vector<__half>& out) {
        out.resize(n);
        return cudaMemcpy(out.data(), b.p, n * sizeof(__half), cudaMemcpyDeviceToHost);
    };
    std::vector<__half> g_h, g_gv, g_y, g_dgv, g_dx, g_dw3, g_dw12;
    CUDA_OK(fetch(d_h, M * F, g_h));
    CUDA_OK(fetch(d_gv, M * 2 * F, g_gv));
    CUDA_OK(fetch(d_y, M * D, g_y));
    CUDA_OK(fetch(d_dgv, M * 2 * F, g_dgv));
    CUDA_OK(fetch(d_dx, M * D, g_dx));
    CUDA_OK(fetch(d_dw3, D * F, g_dw3));
    CUDA_OK(fetch(d_dw12, 2 * F * D, g_dw12));

    bool ok = true;
    ok &= report("gv", g_gv, t_gv, 1e-2);
    ok &= report("h", g_h, t_h, 1e-2);
    ok &= report("y", g_y, t_y, 1e-2);
    ok &= report("dgv", g_dgv, t_dgv, 1e-2);
    ok &= report("dx", g_dx, t_dx, 1e-2);
    ok &= report("dw3", g_dw3, t_dw3, 1e-2);
    ok &= report("dw12", g_dw12, t_dw12, 1e-2);

    // argument errors come back as status codes, before anything is launched
    const bool refused = mgr_gemm_tn(d_y.p, d_h.p, d_w3.p, M, D, F - 1, F, F, D, MGR_F16, stream) == MGR_ERR_BAD_SHAPE &&
                         mgr_swiglu_fused_fwd_save(d_h.p, d_gv.p, d_x.p, d_w12.p, M, D, F, MGR_F32, stream) == MGR_ERR_BAD_DTYPE &&
                         mgr_swiglu_dh_dgv(nullptr, d_dy.p, d_w3.p, d_gv.p, M, D, F, MGR_F16, stream) == MGR_ERR_NULL_PTR;
    std::printf("argument errors refused: %s\n", refused ? "ok" : "FAILED");
    ok &= refused;

    cudaStreamDestroy(stream);
    std::printf(ok ? "Validation PASSED\n" : "Validation FAILED\n");
    return ok ? 0 : 1;
}
