// Torch-free check of the C ABI: a plain C++ host program that links libmgr_b200.so, runs RMSNorm
// forward and backward through mgr_rmsnorm_fwd / mgr_rmsnorm_bwd / mgr_rmsnorm_bwd_noalloc on the
// shape of the reference's stand-alone test (2048 x 4096 fp32, values uniform in (-1, 1), eps 1e-5,
// forward tolerance 1e-4: rmsnorm_standalone.cu:33-35, 45-49, 75-86) and compares with the CPU
// oracle (mgr_oracle.c, linked in). Prints one line per check and exits non-zero on failure.
//
// Build (from the repository root):
//   nvcc -O2 -std=c++17 -Iinclude tests/standalone/rmsnorm_abi_check.cu oracle/mgr_oracle.c \
//        -Lmgrrmsnorm_b200/lib -lmgr_b200 -Xlinker -rpath=$PWD/mgrrmsnorm_b200/lib -o /tmp/rmsnorm_abi_check
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <random>
#include <vector>

#include "mgr_b200.h"

extern "C" {
void mgr_oracle_rmsnorm_fwd_f64(double* y, double* inv_rms, const float* x, const float* w, int64_t rows, int64_t cols, float eps);
void mgr_oracle_rmsnorm_bwd_f64(double* dx, double* dw, const float* dy, const float* x, const float* w, int64_t rows, int64_t cols, float eps);
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

static double max_abs_diff(const std::vector<float>& got, const std::vector<double>& want) {
    double m = 0;
    for (size_t i = 0; i < got.size(); ++i) m = std::fmax(m, std::fabs(static_cast<double>(got[i]) - want[i]));
    return m;
}

int main() {
    const int64_t rows = 2048, cols = 4096;
    const float eps = 1e-5f;
    const size_t n = static_cast<size_t>(rows) * cols;
    std::mt19937 gen(1234);
    std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
    std::vector<float> x(n), dy(n), w(cols);
    for (auto& v : x) v = dist(gen);
    for (auto& v : w) v = dist(gen);
    for (auto& v : dy) v = dist(gen);

    int sms = 0;
    MGR_OK_OR_DIE(mgr_device_check(&sms));
    std::printf("abi version %d, %d SMs\n", mgr_abi_version(), sms);

    float *d_x, *d_dy, *d_w, *d_y, *d_dx, *d_dx2, *d_dw, *d_dw2, *d_inv;
    void* d_ws;
    CUDA_OK(cudaMalloc(&d_x, n * 4));
    CUDA_OK(cudaMalloc(&d_dy, n * 4));
    CUDA_OK(cudaMalloc(&d_y, n * 4));
    CUDA_OK(cudaMalloc(&d_dx, n * 4));
    CUDA_OK(cudaMalloc(&d_dx2, n * 4));
    CUDA_OK(cudaMalloc(&d_w, cols * 4));
    CUDA_OK(cudaMalloc(&d_dw, cols * 4));
    CUDA_OK(cudaMalloc(&d_dw2, cols * 4));
    CUDA_OK(cudaMalloc(&d_inv, rows * 4));
    const size_t ws_bytes = mgr_rmsnorm_bwd_workspace_bytes(rows, cols, MGR_F32);
    CUDA_OK(cudaMalloc(&d_ws, ws_bytes));
    CUDA_OK(cudaMemcpy(d_x, x.data(), n * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_dy, dy.data(), n * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(d_w, w.data(), cols * 4, cudaMemcpyHostToDevice));

    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    MGR_OK_OR_DIE(mgr_rmsnorm_fwd(d_y, d_inv, d_x, d_w, rows, cols, eps, MGR_F32, stream));
    MGR_OK_OR_DIE(mgr_rmsnorm_bwd(d_dx, d_dw, nullptr, d_dy, d_x, d_w, d_inv, rows, cols, MGR_F32, d_ws, ws_bytes, stream));
    MGR_OK_OR_DIE(mgr_rmsnorm_bwd_noalloc(d_dx2, d_dw2, nullptr, d_dy, d_x, d_w, d_inv, rows, cols, MGR_F32, stream));
    CUDA_OK(cudaStreamSynchronize(stream));
    MGR_OK_OR_DIE(mgr_device_status(1));

    std::vector<float> y(n), dx(n), dx2(n), dw(cols), dw2(cols);
    CUDA_OK(cudaMemcpy(y.data(), d_y, n * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(dx.data(), d_dx, n * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(dx2.data(), d_dx2, n * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(dw.data(), d_dw, cols * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(dw2.data(), d_dw2, cols * 4, cudaMemcpyDeviceToHost));

    std::vector<double> ty(n), tdx(n), tdw(cols);
    mgr_oracle_rmsnorm_fwd_f64(ty.data(), nullptr, x.data(), w.data(), rows, cols, eps);
    mgr_oracle_rmsnorm_bwd_f64(tdx.data(), tdw.data(), dy.data(), x.data(), w.data(), rows, cols, eps);

    int bad = 0;
    const double e_y = max_abs_diff(y, ty), e_dx = max_abs_diff(dx, tdx), e_dw = max_abs_diff(dw, tdw);
    std::printf("forward  max |y  - oracle| = %.3e  (limit 1e-4)  %s\n", e_y, e_y < 1e-4 ? "ok" : "FAILED");
    std::printf("backward max |dx - oracle| = %.3e  (limit 1e-4)  %s\n", e_dx, e_dx < 1e-4 ? "ok" : "FAILED");
    std::printf("backward max |dw - oracle| = %.3e  (limit 1e-3)  %s\n", e_dw, e_dw < 1e-3 ? "ok" : "FAILED");
    bad += !(e_y < 1e-4) + !(e_dx < 1e-4) + !(e_dw < 1e-3);
    bool same = true;
    for (size_t i = 0; i < n && same; ++i) same = dx[i] == dx2[i];
    for (int64_t j = 0; j < cols && same; ++j) same = dw[j] == dw2[j];
    std::printf("allocation-free backward equals the workspace backward bit for bit: %s\n", same ? "ok" : "FAILED");
    bad += !same;
    std::printf(bad ? "Validation FAILED\n" : "Validation PASSED\n");
    return bad ? 1 : 0;
}
