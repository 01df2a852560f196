/*
 * mgr_b200.h -- C ABI of libmgr_b200.so: sm_100a (B200) kernels for the two MegaGemm hot paths,
 * RMSNorm forward/backward and the SwiGLU MLP.
 *
 * This is the boundary a maintainer of the reference binds instead of its own kernel library:
 * the typed C++ wrappers of src/rmsnorm_kernel.h:9-67 (called from pytorch_binding/binding.cpp:36-59,
 * 96-126) and the Triton launches of megagemm/swiglu.py:103-107,125-129.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer on the current CUDA device
 *     unless the comment says "host";
 *   - `dtype` is one of MGR_F32 / MGR_F16 / MGR_BF16 and applies to every `void*` tensor of the call
 *     (the reference has the same one-dtype-per-call contract, binding.cpp:34-63);
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream, which is what
 *     the reference always uses, src/rmsnorm_kernel.cu:542);
 *   - the library allocates nothing, frees nothing, never synchronises the device, never prints;
 *     outputs and scratch are caller-owned (the reference's binding allocates outputs through
 *     torch the same way, binding.cpp:29-30,89-90);
 *   - return value: MGR_OK (0) or a negative MGR_ERR_* code; mgr_status_str() names it. Argument
 *     errors are detected on the host before anything is launched (the reference returns `false`
 *     after an fprintf, src/rmsnorm_kernel.cu:533-549).
 *   - tensors are row-major and dense: row r of an [rows, cols] tensor starts at element r*cols.
 *   - threads: every entry point may be called from several host threads at once (on the same or on
 *     different devices and streams). The only state the library keeps is per-device facts it looks up
 *     once (SM count, occupancy, kernel attributes, symbol addresses), held in atomics, plus two
 *     process-wide settings the caller owns: mgr_gemm_set_sm_limit and the shared scratch of
 *     mgr_rmsnorm_bwd_noalloc (see there). The reference keeps no state either
 *     (src/rmsnorm_kernel.cu has no globals).
 */
#ifndef MGR_B200_H_
#define MGR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MGR_ABI_VERSION 1

/* element types (reference: fp32 / fp16 / bf16 kernel families, src/rmsnorm_kernel.h:9-67) */
#define MGR_F32 0
#define MGR_F16 1
#define MGR_BF16 2

/* status codes */
#define MGR_OK 0
#define MGR_ERR_BAD_DTYPE (-1)
#define MGR_ERR_BAD_SHAPE (-2)
#define MGR_ERR_NULL_PTR (-3)
#define MGR_ERR_MISALIGNED (-4)
#define MGR_ERR_WORKSPACE_TOO_SMALL (-5)
#define MGR_ERR_UNSUPPORTED_ARCH (-6)
#define MGR_ERR_LAUNCH_FAILED (-7)
#define MGR_ERR_DEVICE_TIMEOUT (-8)
#define MGR_ERR_TOO_LARGE (-9)
#define MGR_ERR_CUDA (-10)

/* Version of this ABI (MGR_ABI_VERSION of the library that was loaded). No reference counterpart. */
int mgr_abi_version(void);

/* Static, NUL-terminated name of a status code. Replaces the reference's stderr messages
 * (src/rmsnorm_kernel.cu:534,538,546). Host pointer; never NULL. */
const char* mgr_status_str(int status);

/* Re-reads the MGR_* environment variables that pin kernel choices for measurements and tests
 * (MGR_RMSNORM_PATH, MGR_RMSNORM_FWD_SHAPE, MGR_RMSNORM_BWD_SHAPE, MGR_RMSNORM_BWD_FAT, MGR_RMSNORM_PREFETCH,
 * MGR_GEMM_CTA_GROUP, MGR_GEMM_PDL, MGR_GEMM_NARROW). The library reads them once, at its first launch, so that no call pays
 * for getenv; a process that changes them afterwards calls this. No reference counterpart (the reference
 * has no environment switches). */
void mgr_reload_env(void);

/* Number of SMs of the current device and whether it can run this library (compute capability 10.x).
 * Returns MGR_OK or MGR_ERR_UNSUPPORTED_ARCH / MGR_ERR_CUDA; *sm_count (host pointer, may be NULL)
 * receives the SM count. No reference counterpart (the reference never asks the device). */
int mgr_device_check(int* sm_count);

/* Status the kernels themselves left on the current device: MGR_OK, or MGR_ERR_DEVICE_TIMEOUT if a
 * bounded wait inside a kernel (an mbarrier wait of a bulk-copy or tensor-core pipeline) ran out since
 * the last clearing read. clear != 0 resets it. This is the ONLY entry point that synchronises (it
 * copies one word from the device); the launch entry points never do. No reference counterpart: the
 * reference's kernels have no device-side waits and its wrappers only see launch errors
 * (src/rmsnorm_kernel.cu:544-548). */
int mgr_device_status(int clear);

/* Test hook: writes `value` into the status word that the kernels of one family set when a bounded wait runs
 * out (family 0: the RMSNorm bulk-copy ring kernels; 1: the tensor-core GEMM kernels), from the host, with a
 * plain copy to the device. It lets a host test walk the path "a kernel gave up -> mgr_device_status reports
 * MGR_ERR_DEVICE_TIMEOUT once -> cleared" without making any kernel wait. Synchronises like mgr_device_status.
 * No reference counterpart. */
int mgr_debug_poke_device_status(int family, int value);

/* ------------------------------------------------------------------------------------------------
 * RMSNorm forward.   y[r,j] = round_dtype((x[r,j] * inv[r]) * w[j]),  inv[r] = 1/sqrt(mean_j x[r,j]^2 + eps)
 *
 * Replaces rmsnorm_cuda_fp32 / _fp16 / _bf16 (src/rmsnorm_kernel.cu:529-550, 577-594, 621-638) and
 * the kernels they launch (src/rmsnorm_kernel.cu:42-230). Arithmetic is fp32 with one rounding to
 * `dtype` on store, as there (:164, :228).
 *   y        [rows, cols] out
 *   inv_rms  [rows] fp32 out, may be NULL (the reference kernel skips the store on NULL, :83)
 *   x        [rows, cols] in;  w [cols] in
 * Accepts every shape the reference accepts (cols%4==0 for fp32, cols%2==0 for fp16/bf16) and, as a
 * superset, any cols >= 1 and any element-aligned pointers (unaligned or odd shapes take a slower
 * scalar kernel instead of being refused). rows == 0 is a no-op.
 */
int mgr_rmsnorm_fwd(void* y, float* inv_rms, const void* x, const void* w,
                    int64_t rows, int64_t cols, float eps, int dtype, void* stream);

/* Row scales alone: inv_rms[r] = 1/sqrt(mean_j x[r,j]^2 + eps), the same kernels as mgr_rmsnorm_fwd with the
 * output stores left out, hence the same bits as the inv_rms that call writes. One read of x, nothing else.
 * It is the first half of an RMSNorm folded into the GEMM that consumes it (mgr_swiglu_fused_fwd_scaled); the
 * reference always materialises the normalised tensor (megagemm/rmsnorm.py:74-75 then megagemm/swiglu.py:167),
 * so it has no counterpart there. */
int mgr_rms_inv(float* inv_rms, const void* x, int64_t rows, int64_t cols, float eps, int dtype, void* stream);

/* Scratch bytes mgr_rmsnorm_bwd needs for this problem on the current device (per-CTA fp32 partial
 * sums of dW). Returns 0 on invalid arguments. Host-only; no reference counterpart (the reference
 * accumulates dW with atomics into the output, src/rmsnorm_kernel.cu:315-325). */
size_t mgr_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t cols, int dtype);

/* RMSNorm backward.
 *   c[r]    = sum_j dy[r,j]*w[j]*x[r,j]
 *   dx[r,j] = round_dtype(inv[r] * (dy[r,j]*w[j] - x[r,j] * c[r]*inv[r]^2/cols))
 *   dw[j]   = round_dtype(sum_r dy[r,j]*x[r,j]*inv[r])          (fp32 sum, ONE rounding)
 *
 * Replaces rmsnorm_backward_cuda_fp32 / _fp16 / _bf16 (src/rmsnorm_kernel.cu:552-574, 596-618,
 * 640-662) and their kernels (:235-522). Differences from the reference, all deliberate:
 *   - dw is a fixed-order fp32 reduction (per-CTA partials in `workspace`, then a column reduce),
 *     so it is bit-reproducible run to run; the reference uses atomicAdd (:319-322) and, for
 *     fp16/bf16, half-precision atomics of rounded partials (:421-422, :517-518);
 *   - every column of dw is produced for every supported cols (the reference leaves dw[8192:]
 *     at zero for fp16/bf16, :344,:371-375);
 *   - dw is fully overwritten; no pre-zeroing is needed (the reference memsets it, :562).
 *   dx [rows, cols] out;  dw [cols] out in `dtype`, may be NULL
 *   dw_f32 [cols] fp32 out, may be NULL: the same sum before the rounding (what a multi-GPU caller
 *          all-reduces before casting). dw and dw_f32 must not both be NULL.
 *   dy, x [rows, cols] in;  w [cols] in;  inv_rms [rows] fp32 in (as written by mgr_rmsnorm_fwd)
 *   workspace / workspace_bytes: >= mgr_rmsnorm_bwd_workspace_bytes(rows, cols, dtype), 16-byte aligned.
 * rows == 0 writes zeros to dw / dw_f32.
 */
int mgr_rmsnorm_bwd(void* dx, void* dw, float* dw_f32, const void* dy, const void* x, const void* w,
                    const float* inv_rms, int64_t rows, int64_t cols, int dtype,
                    void* workspace, size_t workspace_bytes, void* stream);

/* RMSNorm backward without a caller-provided workspace. It has no counterpart in the reference (whose
 * backward needs no scratch because it accumulates dW with atomics, src/rmsnorm_kernel.cu:315-325).
 *
 * Same arguments, arithmetic, kernels and results as mgr_rmsnorm_bwd, minus `workspace`: the partial
 * rows of dW go to a fixed MGR_NOALLOC_SCRATCH_BYTES array inside the library's device image. It is for
 * hosts that cannot obtain device memory at call time: a C/C++ program without a stream-ordered
 * allocator, or a running service that keeps cudaMalloc/cudaFree out of its steady state because both
 * synchronise the device and may fail once memory is fragmented. The call itself allocates nothing
 * (no cudaMalloc, no cudaFree, no allocating library routine).
 *   - Limit: problems whose mgr_rmsnorm_bwd_workspace_bytes(rows, cols, dtype) exceeds
 *     MGR_NOALLOC_SCRATCH_BYTES return MGR_ERR_TOO_LARGE ("dimension exceeds the supported maximum": here the
 *     maximum is this scratch size) before anything is launched. The need is one fp32 row of `cols` per CTA of
 *     the backward kernel, i.e. cols * 4 * (SM count x resident CTAs of the kernel chosen for that row length),
 *     so it is a property of the device: on a 148-SM B200 every row length up to 16384 columns fits whatever
 *     the dtype and row count (largest: 9.25 MiB at fp32 x 16384 columns; a test sweeps every multiple of 8);
 *     fp16/bf16 rows of 32768 columns, whose kernels write 148 partial rows of 128 KiB, do not.
 *   - Every GPU whose context loads the library holds the array until the process ends.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, once per
 *     device, with that device current). Make that first call before starting any stream capture.
 *   - All calls on a device share the array; it keeps the last call's contents and needs no clearing.
 *     Calls that may overlap on the GPU (different streams without an ordering) race: serialise them.
 */
#define MGR_NOALLOC_SCRATCH_BYTES (16u << 20)
int mgr_rmsnorm_bwd_noalloc(void* dx, void* dw, float* dw_f32, const void* dy, const void* x, const void* w,
                            const float* inv_rms, int64_t rows, int64_t cols, int dtype, void* stream);

/* Residual add fused into the norm, the pair of operations that opens a pre-norm transformer block:
 *   h = x + residual;  y = RMSNorm(h) * w.
 * The reference has no fused form; it replaces the sequence a caller of the reference writes as
 * `h = x + residual` (a torch elementwise kernel) followed by RMSNormFunction.forward
 * (megagemm/rmsnorm.py:22-36), and gives the same bits as that sequence run through mgr_rmsnorm_fwd:
 * h is rounded to `dtype` first and the norm is taken of the rounded h.
 *   y [rows, cols] out;  h [rows, cols] out (may be the buffer of x or of residual: in-place update of
 *   the residual stream);  inv_rms [rows] fp32 out, may be NULL;  x, residual [rows, cols] in;  w [cols] in.
 * Four passes over [rows, cols] (reads x, residual; writes h, y) instead of the five of the two-step
 * sequence.
 */
int mgr_add_rmsnorm_fwd(void* y, void* h, float* inv_rms, const void* x, const void* residual, const void* w,
                        int64_t rows, int64_t cols, float eps, int dtype, void* stream);

/* Backward of the above: dh = dRMSNorm(h; dy) + dres, where dres is the gradient arriving along the
 * residual stream (the gradient of whatever else consumed h). dh is at once the gradient of x and of
 * residual. One rounding of the fp32 sum, where the two-step sequence (RMSNormFunction.backward,
 * megagemm/rmsnorm.py:39-48, then autograd's accumulation of the two gradients of h) rounds twice.
 *   dh [rows, cols] out (may be the buffer of dres);  dw, dw_f32, workspace as for mgr_rmsnorm_bwd (same
 *   workspace size);  dy, dres, h [rows, cols] in;  w [cols] in;  inv_rms [rows] fp32 in.
 */
int mgr_add_rmsnorm_bwd(void* dh, void* dw, float* dw_f32, const void* dy, const void* dres, const void* h,
                        const void* w, const float* inv_rms, int64_t rows, int64_t cols, int dtype,
                        void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------------
 * SwiGLU activation on an already-projected tensor: gv = [gate | val] of shape [m, 2f] (gate =
 * columns [0,f), val = columns [f,2f): the layout nn.Linear(d, 2*hidden) produces and
 * benchmark_swiglu.py:85-89 fills).
 *   forward : h[r,j]   = round_dtype(gate*sigmoid(gate)*val)                         h [m, f]
 *   backward: dgv[r,j] = round_dtype(dh*val*sig*(1 + gate*(1 - sig)))   (d_gate)     dgv [m, 2f]
 *             dgv[r,f+j] = round_dtype(dh*gate*sig)                     (d_val)
 * Replace the Triton kernels _mg_swiglu_fwd_kernel / _mg_swiglu_bwd_kernel and their launches in
 * MegaGemmFunction (megagemm/swiglu.py:18-43, 46-79, 103-107, 125-129). fp32 math, one rounding.
 * Any f >= 1; m == 0 is a no-op.
 */
int mgr_swiglu_act_fwd(void* h, const void* gv, int64_t m, int64_t f, int dtype, void* stream);
int mgr_swiglu_act_bwd(void* dgv, const void* dh, const void* gv, int64_t m, int64_t f, int dtype, void* stream);

/* ------------------------------------------------------------------------------------------------
 * SwiGLU MLP on tensor cores (tcgen05 / TMEM / TMA). fp16 and bf16 only, fp32 accumulation.
 *
 * mgr_swiglu_fused_fwd: h[m, f] = round_dtype( silu(x w12[0:f]^T) * (x w12[f:2f]^T) ) in one kernel.
 *   x [m, d] row-major; w12 [2f, d] row-major with the gate rows first and the value rows second (the
 *   layout of MegaGemmTriton.w12.weight, megagemm/swiglu.py:163, benchmark_swiglu.py:85-89).
 *   Replaces `self.w12(x)` followed by MegaGemmFunction (megagemm/swiglu.py:167-168): the [m, 2f]
 *   projection is never written to memory, and the activation sees the fp32 accumulator instead of a
 *   value already rounded to fp16/bf16.
 * mgr_gemm_tn: c[m, n] = round_dtype( a[m, k] b[n, k]^T ), leading dimensions in elements. Replaces an
 *   nn.Linear without bias (`self.w3(hidden)`, megagemm/swiglu.py:169).
 * Requirements: d, f, n, k and the leading dimensions multiples of 8; pointers 16-byte aligned.
 * m == 0 is a no-op. Shapes outside these limits return MGR_ERR_BAD_SHAPE (the caller then keeps
 * the library GEMM it would have used with the reference).
 */
int mgr_swiglu_fused_fwd(void* h, const void* x, const void* w12, int64_t m, int64_t d, int64_t f, int dtype, void* stream);

/* mgr_swiglu_fused_fwd with a scale per row applied to both halves of the projection before the activation:
 *   h[r, :] = silu(s_r * (x[r] w12[0:f]^T)) * (s_r * (x[r] w12[f:2f]^T)),   s = row_scale [m] fp32 (NULL = all ones).
 * With s = mgr_rms_inv(x) and w12 = w12_original * w_norm (each column k scaled by the norm weight w_norm[k], folded
 * once by the caller) this is the pre-norm block's `w12(norm(x))` + activation (megagemm/rmsnorm.py:74-75,
 * megagemm/swiglu.py:167-168) without the normalised [m, d] tensor ever being written or read: an inference-time
 * form (the folded weight is only valid while w_norm and w12 do not change). */
int mgr_swiglu_fused_fwd_scaled(void* h, const void* x, const void* w12, const float* row_scale, int64_t m, int64_t d,
                                int64_t f, int dtype, void* stream);
int mgr_gemm_tn(void* c, const void* a, const void* b, int64_t m, int64_t n, int64_t k,
                int64_t lda, int64_t ldb, int64_t ldc, int dtype, void* stream);

/* The backward GEMMs of the MLP. The reference gets them from autograd of its two nn.Linear layers
 * (Linear(w3).backward and Linear(w12).backward, implicit after megagemm/swiglu.py:167,169) and its
 * Triton backward kernel (megagemm/swiglu.py:111-131); here they are the same tensor-core kernel family.
 *
 * mgr_gemm: c[m, n] = round_dtype( op(a) op(b)^T ) where each operand is stored either K-major
 *   (a: [m, k] row-major, b: [n, k] row-major; *_mn_major = 0) or MN-major (a: [k, m] row-major,
 *   b: [k, n] row-major; *_mn_major = 1). lda / ldb are the row pitches of the stored matrices in
 *   elements. So, with dy [M, D], h [M, F], dgv [M, 2F], x [M, D], w3 [D, F], w12 [2F, D]:
 *     dh   = dy w3       : mgr_gemm(dh,   dy,  w3,  M,  F, D,  ..., 0, 1)
 *     dw3  = dy^T h      : mgr_gemm(dw3,  dy,  h,   D,  F, M,  ..., 1, 1)
 *     dx   = dgv w12     : mgr_gemm(dx,   dgv, w12, M,  D, 2F, ..., 0, 1)
 *     dw12 = dgv^T x     : mgr_gemm(dw12, dgv, x,   2F, D, M,  ..., 1, 1)
 *   No operand is ever transposed in memory. m (for an MN-major a), n and k multiples of 8.
 * mgr_swiglu_fused_bwd: dgv[m, 2f] = [d_gate | d_val] from dh[m, f], recomputing the projection
 *   x w12^T tile by tile in TMEM (it is not stored by the forward):
 *     d_val = dh*gate*sig(gate),  d_gate = dh*val*sig(gate)*(1 + gate*(1 - sig(gate)))
 *   i.e. `w12(x)` recomputed + _mg_swiglu_bwd_kernel (megagemm/swiglu.py:46-79) in one kernel.
 */
int mgr_gemm(void* c, const void* a, const void* b, int64_t m, int64_t n, int64_t k, int64_t lda, int64_t ldb,
             int64_t ldc, int a_mn_major, int b_mn_major, int dtype, void* stream);
int mgr_swiglu_fused_bwd(void* dgv, const void* dh, const void* x, const void* w12, int64_t m, int64_t d, int64_t f,
                         int dtype, void* stream);

/* The same forward/backward pair when the projection IS kept for backward, as the reference keeps
 * w12_out (ctx.save_for_backward, megagemm/swiglu.py:98): one store of [m, 2f] in forward instead of a
 * second projection GEMM in backward.
 * mgr_swiglu_fused_fwd_save: mgr_swiglu_fused_fwd that also writes gv[m, 2f] = round_dtype([gate | val]).
 *   h is still computed from the fp32 accumulators, not from the rounded gv.
 * mgr_swiglu_dh_dgv: dgv[m, 2f] = [d_gate | d_val] from dy[m, d], w3[d, f] and the stored gv: the GEMM
 *   dh = dy w3 (Linear(w3).backward) with _mg_swiglu_bwd_kernel (megagemm/swiglu.py:46-79) as its
 *   epilogue; dh stays in fp32 in tensor memory and is never written.
 */
int mgr_swiglu_fused_fwd_save(void* h, void* gv, const void* x, const void* w12, int64_t m, int64_t d, int64_t f,
                              int dtype, void* stream);
int mgr_swiglu_dh_dgv(void* dgv, const void* dy, const void* w3, const void* gv, int64_t m, int64_t d, int64_t f,
                      int dtype, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Cross-rank sum of a short fp32 vector over NVLink peer memory (one process per GPU): the dW of a row-sharded
 * RMSNorm, summed in fp32 across the ranks and rounded once. The reference has no distributed code, so this has no
 * counterpart there; it replaces the NCCL all-reduce the multi-GPU layer of this library used first, which for a
 * 32 KB vector is pure latency (18 us on 2-4 GPUs, 55 us on 8).
 *
 * Every rank owns one buffer of mgr_peer_allreduce_buffer_bytes(world, n_max) bytes that EVERY rank can write
 * (peer-mapped: torch symmetric memory, CUDA IPC or cuMem exports all do), zero-filled before the first call,
 * 256-byte aligned. `peer_buffers` is a HOST array of `world` device pointers: entry q is rank q's buffer as mapped
 * in the calling process (entry `rank` is the caller's own). `calls` is MGR_PEER_ALLREDUCE_CTAS uint32 counters in
 * the caller's own device memory, zero-filled once; the kernel keeps its call number there, so a captured graph
 * replays correctly. One launch per rank: stores this rank's `src[n]` into every rank's buffer (each value paired
 * with the call's number in one 8-byte store, so no fence or flag is needed), waits on the elements of every rank as
 * they arrive in its own, adds them in rank order (the same order, hence the same bits, on every rank) and writes
 * out_f32[n] (may be NULL) and out[n] in `dtype` (may be NULL; not both).
 *   n a multiple of 4, n <= n_max; all ranks call with the same n, in the same order, once per step each.
 * The wait is bounded (about a second); if a rank never arrives the kernel returns, leaves the outputs unwritten and
 * mgr_device_status() reports MGR_ERR_DEVICE_TIMEOUT. Only peer STORES and local loads are used. */
#define MGR_PEER_ALLREDUCE_CTAS 16
size_t mgr_peer_allreduce_buffer_bytes(int world, int64_t n_max);
int mgr_peer_allreduce_f32(const void* const* peer_buffers, int rank, int world, const float* src, float* out_f32,
                           void* out, int dtype, int64_t n, int64_t n_max, void* calls, void* stream);

/* Limits the GEMM kernels of this process to `sms` SMs (0 = all of them); returns the previous limit.
 * The GEMM kernels are persistent (one CTA per SM), so a collective launched beside one finds no free SM
 * unless some are left out: a tensor-parallel caller lowers the limit around the GEMMs it overlaps with an
 * all-reduce and restores it afterwards. Host-side setting, read at each launch. No reference counterpart
 * (the reference has no distributed code). */
int mgr_gemm_set_sm_limit(int sms);

#ifdef __cplusplus
}
#endif
#endif /* MGR_B200_H_ */
