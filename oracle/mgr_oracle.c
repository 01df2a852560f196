/*
 * mgr_oracle.c -- CPU restatement of the reference's arithmetic for its two hot paths.
 *
 * TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA kernels are compared against; it is
 * never on the product path (only tests, the smoke check and the benchmark's CPU-baseline leg load it).
 *
 * Inputs are fp32 arrays whose values are already exactly representable in the dtype under test
 * (the caller rounds to fp16/bf16 first), so one set of functions serves all three dtypes.
 * Two flavours:
 *   *_f64  : every sum and product in double -- the ground truth a kernel's output is judged against;
 *   *_f32seq: the reference's own fp32 evaluation order where it has CPU code (forward only),
 *             so it can be pinned bit-for-bit against that code compiled from the reference tree.
 *
 * Build: see oracle/Makefile (gcc -O2 -fopenmp, no -ffast-math).
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int mgr_oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Forward, ground truth.
 * Follows src/rmsnorm_kernel.cu:56-101 (sum of squares :60-66, inv = rsqrt(sum/cols + eps) :82,
 * y = x*inv*w :95-98); the formula is also test_rmsnorm.py:55-56. eps is the fp32 value the kernel
 * receives, widened. */
void mgr_oracle_rmsnorm_fwd_f64(double* y, double* inv_rms, const float* x, const float* w,
                                int64_t rows, int64_t cols, float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < rows; ++r) {
        const float* xr = x + r * cols;
        double ss = 0.0;
        for (int64_t j = 0; j < cols; ++j) ss += (double)xr[j] * (double)xr[j];
        const double inv = 1.0 / sqrt(ss / (double)cols + (double)eps);
        if (inv_rms) inv_rms[r] = inv;
        if (y)
            for (int64_t j = 0; j < cols; ++j) y[r * cols + j] = (double)xr[j] * inv * (double)w[j];
    }
}

/* Forward in the reference's CPU evaluation order: sequential fp32 sum, 1/sqrtf, (x*rms)*w.
 * Follows rmsnorm_cpu, rmsnorm_standalone.cu:17-30. */
void mgr_oracle_rmsnorm_fwd_f32seq(float* y, const float* x, const float* w, int64_t rows, int64_t cols, float eps) {
    for (int64_t r = 0; r < rows; ++r) {
        float ss = 0.0f;
        for (int64_t j = 0; j < cols; ++j) {
            const float v = x[r * cols + j];
            ss += v * v;
        }
        const float rms = 1.0f / sqrtf(ss / cols + eps);
        for (int64_t j = 0; j < cols; ++j) y[r * cols + j] = x[r * cols + j] * rms * w[j];
    }
}

/* Backward, ground truth. inv_rms is recomputed in double from x (so the oracle does not inherit a
 * kernel's fp32 inv_rms).
 *   c   = sum_j dy*w*x                       src/rmsnorm_kernel.cu:267-270
 *   dx  = inv*(dy*w - x*c*inv^2/cols)        src/rmsnorm_kernel.cu:298, 306-309
 *   dw_j = sum_r dy*x*inv                    src/rmsnorm_kernel.cu:272-277
 * dw is summed over rows in increasing r per column (double). */
void mgr_oracle_rmsnorm_bwd_f64(double* dx, double* dw, const float* dy, const float* x, const float* w,
                                int64_t rows, int64_t cols, float eps) {
    for (int64_t j = 0; j < cols; ++j) dw[j] = 0.0;
#pragma omp parallel
    {
        double* local = 0;
#pragma omp critical
        { local = (double*)__builtin_malloc((size_t)cols * sizeof(double)); }
        for (int64_t j = 0; j < cols; ++j) local[j] = 0.0;
#pragma omp for schedule(static)
        for (int64_t r = 0; r < rows; ++r) {
            const float* xr = x + r * cols;
            const float* gr = dy + r * cols;
            double ss = 0.0, c = 0.0;
            for (int64_t j = 0; j < cols; ++j) {
                ss += (double)xr[j] * (double)xr[j];
                c += (double)gr[j] * (double)w[j] * (double)xr[j];
            }
            const double inv = 1.0 / sqrt(ss / (double)cols + (double)eps);
            const double term2 = c * inv * inv / (double)cols;
            for (int64_t j = 0; j < cols; ++j) {
                if (dx) dx[r * cols + j] = inv * ((double)gr[j] * (double)w[j] - (double)xr[j] * term2);
                local[j] += (double)gr[j] * (double)xr[j] * inv;
            }
        }
#pragma omp critical
        {
            for (int64_t j = 0; j < cols; ++j) dw[j] += local[j];
            __builtin_free(local);
        }
    }
}

/* SwiGLU activation forward: h = gate*sigmoid(gate)*val, gate = gv[:, :F], val = gv[:, F:].
 * Follows _mg_swiglu_fwd_kernel, megagemm/swiglu.py:35-41. */
void mgr_oracle_swiglu_act_fwd_f64(double* h, const float* gv, int64_t m, int64_t f) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < m; ++r)
        for (int64_t j = 0; j < f; ++j) {
            const double g = gv[r * 2 * f + j], v = gv[r * 2 * f + f + j];
            const double sig = 1.0 / (1.0 + exp(-g));
            h[r * f + j] = g * sig * v;
        }
}

/* SwiGLU activation backward: writes [d_gate | d_val] as [m, 2f].
 *   d_val  = dh*gate*sig ;  d_gate = dh*val*sig*(1 + gate*(1 - sig))
 * Follows _mg_swiglu_bwd_kernel, megagemm/swiglu.py:64-76. */
void mgr_oracle_swiglu_act_bwd_f64(double* dgv, const float* dh, const float* gv, int64_t m, int64_t f) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < m; ++r)
        for (int64_t j = 0; j < f; ++j) {
            const double g = gv[r * 2 * f + j], v = gv[r * 2 * f + f + j], go = dh[r * f + j];
            const double sig = 1.0 / (1.0 + exp(-g));
            dgv[r * 2 * f + j] = go * v * (sig * (1.0 + g * (1.0 - sig)));
            dgv[r * 2 * f + f + j] = go * (g * sig);
        }
}

/* C[m,n] = sum_k A[m,k]*B[n,k] in double: the contraction of nn.Linear without bias
 * (megagemm/swiglu.py:163-169: w12(x), w3(h)). Small sizes only (naive loops). */
void mgr_oracle_linear_f64(double* c, const float* a, const float* b, int64_t m, int64_t n, int64_t k) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            double s = 0.0;
            for (int64_t t = 0; t < k; ++t) s += (double)a[i * k + t] * (double)b[j * k + t];
            c[i * n + j] = s;
        }
}
