// RMSNorm kernels fed by a shared-memory ring of bulk asynchronous copies (1-D TMA).
//
// One persistent CTA per SM. A producer warp keeps `nslots` row blocks in flight with
// cp.async.bulk (global -> shared, completion on an mbarrier); consumer warps work out of shared
// memory and write results straight to global. Loads therefore never wait for compute and the bytes
// in flight per SM are set by the ring depth, not by registers -- which is what a 16-32 KB row needs
// to keep HBM3e busy. x (and dy) cross HBM exactly once per direction.
//
// One CTA per SM, each issuing its own copies. Every mbarrier wait is bounded (mgr_ptx.cuh); a timeout raises the CTA's
// abort flag, sets *status and lets all roles fall out of their loops.
#pragma once

#include "mgr_common.cuh"
#include "mgr_ptx.cuh"

namespace mgr {

constexpr int kRingMaxSlots = 16;
constexpr int kFwdRingWarps = 8;  // consumer warps of the forward ring kernel
constexpr uint32_t kSmemBudget = 225u * 1024u;  // dynamic shared memory asked for; 227 KB per CTA on sm_100 includes the static part

struct RingPlan {
    int ok;             // 0: shape does not fit the ring path
    int nslots;         // ring depth
    int rows_per_slot;  // rows one bulk copy brings in
    uint32_t slot_bytes;
    uint32_t w_bytes;   // forward only: shared copy of the weight row
    uint32_t smem_bytes;
};

// ------------------------------------------------------------------------------------------------
// Forward: warp per row. Chunk i of this CTA's chunk sequence lives in slot i % nslots and is consumed
// by warp i % ncw, where ncw = min(NCW, nslots) and nslots is a multiple of ncw -- so a slot always
// belongs to the same warp. That matters: a warp only ever waits for the NEXT fill of its own slots.
// (If slots rotated among warps, a fast warp could wait for fill u+1 of a slot whose fill u is still
// in flight, and an mbarrier parity wait cannot tell phase u-1 "done" from phase u+1 "done".)
// Shared memory: [ w | slot 0 .. slot n-1 | full[n] empty[n] ].
// ------------------------------------------------------------------------------------------------

template <typename T, int NCW>
__global__ void __launch_bounds__((NCW + 1) * 32, 1)
rms_fwd_ring(T* __restrict__ y, float* __restrict__ inv_rms, const T* __restrict__ x, const T* __restrict__ w,
             int64_t rows, int cols, float eps, int rows_per_slot, int nslots, uint32_t w_bytes, uint32_t slot_bytes,
             int* __restrict__ status) {
    constexpr int VEC = Elem<T>::kVec;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int abort_flag;
    const uint32_t s_w = ptx::smem_addr(smem);
    const uint32_t s_slots = s_w + w_bytes;
    const uint32_t s_full = s_slots + static_cast<uint32_t>(nslots) * slot_bytes;
    const uint32_t s_empty = s_full + 8u * nslots;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = cols / VEC;
    const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
    const int64_t nchunks = (rows + rows_per_slot - 1) / rows_per_slot;
    const int64_t my_chunks = blockIdx.x < nchunks ? (nchunks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < nslots; ++s) {
            ptx::mbar_init(s_full + 8u * s, 1);
            ptx::mbar_init(s_empty + 8u * s, 1);
        }
        ptx::fence_mbar_init();
    }
    // weight row -> shared (generic proxy; read only by the consumers)
    for (int v = threadIdx.x; v < nvec; v += blockDim.x)
        reinterpret_cast<uint4*>(smem)[v] = __ldg(reinterpret_cast<const uint4*>(w) + v);
    __syncthreads();

    if (warp == NCW) {
        // ---- producer ----
        if (lane == 0) {
            for (int64_t i = 0; i < my_chunks; ++i) {
                const int s = static_cast<int>(i % nslots);
                const uint32_t use = static_cast<uint32_t>(i / nslots);
                if (use > 0 && !ptx::mbar_wait(s_empty + 8u * s, (use - 1) & 1u, &abort_flag)) break;
                const int64_t r0 = (blockIdx.x + i * gridDim.x) * rows_per_slot;
                const int64_t live = rows - r0 < rows_per_slot ? rows - r0 : rows_per_slot;
                const uint32_t bytes = static_cast<uint32_t>(live) * row_bytes;
                ptx::mbar_arrive_expect_tx(s_full + 8u * s, bytes);
                ptx::bulk_copy_g2s(s_slots + s * slot_bytes, x + r0 * cols, bytes, s_full + 8u * s);
            }
        }
    } else {
        // ---- consumers ----
        const float inv_cols = 1.0f / static_cast<float>(cols);
        const int ncw = nslots < NCW ? nslots : NCW;
        for (int64_t i = warp; warp < ncw && i < my_chunks; i += ncw) {
            const int s = static_cast<int>(i % nslots);
            const uint32_t use = static_cast<uint32_t>(i / nslots);
            if (!ptx::mbar_wait(s_full + 8u * s, use & 1u, &abort_flag)) break;
            const int64_t r0 = (blockIdx.x + i * gridDim.x) * rows_per_slot;
            const int live = static_cast<int>(rows - r0 < rows_per_slot ? rows - r0 : rows_per_slot);
            for (int rr = 0; rr < live; ++rr) {
                const uint32_t s_row = s_slots + s * slot_bytes + rr * row_bytes;
                float ss = 0.f;
#pragma unroll 4
                for (int v = lane; v < nvec; v += 32) {
                    float f[VEC];
                    unpack16<T>(ptx::lds128(s_row + 16u * v), f);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) ss += f[k] * f[k];
                }
                ss = warp_sum(ss);
                const float inv = 1.0f / sqrtf(ss * inv_cols + eps);
                const int64_t r = r0 + rr;
                if (lane == 0 && inv_rms != nullptr) inv_rms[r] = inv;
                uint4* yr = reinterpret_cast<uint4*>(y + r * cols);
#pragma unroll 4
                for (int v = lane; v < nvec; v += 32) {
                    float f[VEC], g[VEC], o[VEC];
                    unpack16<T>(ptx::lds128(s_row + 16u * v), f);
                    unpack16<T>(ptx::lds128(s_w + 16u * v), g);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) o[k] = (f[k] * inv) * g[k];
                    st_stream16(yr + v, pack16<T>(o));
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(s_empty + 8u * s);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag != 0) atomicExch(status, MGR_ERR_DEVICE_TIMEOUT);
}

inline RingPlan fwd_ring_plan(int64_t rows, int64_t cols, size_t elem) {
    RingPlan p{};
    const uint64_t row_bytes = static_cast<uint64_t>(cols) * elem;
    if (row_bytes % 16 != 0 || row_bytes > 64 * 1024) return p;
    p.w_bytes = static_cast<uint32_t>((row_bytes + 127) / 128 * 128);
    int rps = static_cast<int>(16384 / row_bytes);
    if (rps < 1) rps = 1;
    if (rps > 64) rps = 64;
    p.rows_per_slot = rps;
    p.slot_bytes = static_cast<uint32_t>(rps * row_bytes);
    const uint32_t fixed = p.w_bytes + 2 * 8 * kRingMaxSlots + 256;
    if (fixed + 4ull * p.slot_bytes > kSmemBudget) return p;
    int n = static_cast<int>((kSmemBudget - fixed) / p.slot_bytes);
    if (n > kRingMaxSlots) n = kRingMaxSlots;
    if (n > kFwdRingWarps) n = n / kFwdRingWarps * kFwdRingWarps;  // a slot must always map to the same consumer warp
    p.nslots = n;
    p.smem_bytes = p.w_bytes + n * p.slot_bytes + 2 * 8 * n;
    p.ok = n >= 4;
    (void)rows;
    return p;
}

// ------------------------------------------------------------------------------------------------
// Backward: 512 threads as G = 512/TPR row groups of TPR threads; a thread owns the same VPT packets
// (VPT*VEC columns) of every row its group sees, so dW partials stay in registers. A slot holds G rows
// of x followed by G rows of dy (two bulk copies). Every warp releases a slot as soon as its packets
// are in registers; thread 0 then refills that slot with the row group `nslots` iterations ahead, so
// there is no separate producer warp (16 warps leave each thread 128 registers).
// Shared memory: [ slot 0 .. slot n-1 | full[n] empty[n] ]; the slot area doubles as the fold
// buffer for the G group partials once the ring has drained.
// ------------------------------------------------------------------------------------------------

constexpr int kBwdRingThreads = 512;

template <typename T, int TPR, int VPT>
__global__ void __launch_bounds__(kBwdRingThreads, 1)
rms_bwd_ring(T* __restrict__ dx, float* __restrict__ ws, const T* __restrict__ dy, const T* __restrict__ x,
             const T* __restrict__ w, const float* __restrict__ inv_rms, int64_t rows, int cols, int nslots,
             uint32_t slot_bytes, int* __restrict__ status) {
    constexpr int VEC = Elem<T>::kVec;
    constexpr int G = kBwdRingThreads / TPR;
    constexpr int NW = kBwdRingThreads / 32;
    constexpr int WPR = TPR / 32;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int abort_flag;
    __shared__ float red[2][NW];
    const uint32_t s_slots = ptx::smem_addr(smem);
    const uint32_t s_full = s_slots + static_cast<uint32_t>(nslots) * slot_bytes;
    const uint32_t s_empty = s_full + 8u * nslots;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nvec = cols / VEC;
    const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
    const int64_t ngroups = (rows + G - 1) / G;
    const int64_t my_groups = blockIdx.x < ngroups ? (ngroups - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    // Brings row group i of this CTA into slot i % nslots (thread 0 only).
    auto fill = [&](int64_t i) {
        const int s = static_cast<int>(i % nslots);
        const int64_t r0 = (blockIdx.x + i * gridDim.x) * G;
        const int64_t live = rows - r0 < G ? rows - r0 : G;
        const uint32_t bytes = static_cast<uint32_t>(live) * row_bytes;
        ptx::mbar_arrive_expect_tx(s_full + 8u * s, 2 * bytes);
        ptx::bulk_copy_g2s(s_slots + s * slot_bytes, x + r0 * cols, bytes, s_full + 8u * s);
        ptx::bulk_copy_g2s(s_slots + s * slot_bytes + G * row_bytes, dy + r0 * cols, bytes, s_full + 8u * s);
    };

    if (threadIdx.x == 0) {
        abort_flag = 0;
        for (int s = 0; s < nslots; ++s) {
            ptx::mbar_init(s_full + 8u * s, 1);
            ptx::mbar_init(s_empty + 8u * s, NW);
        }
        ptx::fence_mbar_init();
        for (int64_t i = 0; i < my_groups && i < nslots; ++i) fill(i);
    }
    __syncthreads();

    const int group = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    uint4 wv[VPT];
    float acc[VPT][VEC];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int v = t + k * TPR;
        wv[k] = v < nvec ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int e = 0; e < VEC; ++e) acc[k][e] = 0.f;
    }
    const float inv_cols = 1.0f / static_cast<float>(cols);
    int buf = 0;
    bool dead = false;
    for (int64_t i = 0; i < my_groups; ++i) {
        const int s = static_cast<int>(i % nslots);
        const uint32_t use = static_cast<uint32_t>(i / nslots);
        // A timed-out thread keeps walking the loop (with zeros) so that the barriers below still see
        // all 512 threads; nothing else can block once waits fail fast on abort_flag.
        if (!dead && !ptx::mbar_wait(s_full + 8u * s, use & 1u, &abort_flag)) dead = true;
        const int64_t r = (blockIdx.x + i * gridDim.x) * G + group;
        const bool live = !dead && r < rows;
        const uint32_t s_x = s_slots + s * slot_bytes + group * row_bytes;
        const uint32_t s_g = s_x + G * row_bytes;
        uint4 xv[VPT], gv[VPT];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            const bool on = live && v < nvec;
            xv[k] = on ? ptx::lds128(s_x + 16u * v) : make_uint4(0, 0, 0, 0);
            gv[k] = on ? ptx::lds128(s_g + 16u * v) : make_uint4(0, 0, 0, 0);
            keep_packed(wv[k]);
        }
        __syncwarp();
        if (lane == 0 && !dead) ptx::mbar_arrive(s_empty + 8u * s);  // packets are in registers: slot is free
        if (threadIdx.x == 0 && !dead && i + nslots < my_groups) {
            if (ptx::mbar_wait(s_empty + 8u * s, use & 1u, &abort_flag)) fill(i + nslots);
            else dead = true;
        }
        const float rinv = live ? __ldg(inv_rms + r) : 0.f;

        float c = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            float fx[VEC], fg[VEC], fw[VEC];
            unpack16<T>(xv[k], fx);
            unpack16<T>(gv[k], fg);
            unpack16<T>(wv[k], fw);
#pragma unroll
            for (int e = 0; e < VEC; ++e) {
                c += (fg[e] * fw[e]) * fx[e];
                acc[k][e] += (fg[e] * fx[e]) * rinv;
            }
        }
        c = warp_sum(c);
        if constexpr (WPR > 1) {
            if (lane == 0) red[buf][warp] = c;
            __syncthreads();
            float sum = 0.f;
#pragma unroll
            for (int q = 0; q < WPR; ++q) sum += red[buf][group * WPR + q];
            buf ^= 1;
            c = sum;
        }
        const float term2 = c * (rinv * rinv) * inv_cols;
        if (live) {
            uint4* dr = reinterpret_cast<uint4*>(dx + r * cols);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                if (v < nvec) {
                    float fx[VEC], fg[VEC], fw[VEC], o[VEC];
                    unpack16<T>(xv[k], fx);
                    unpack16<T>(gv[k], fg);
                    unpack16<T>(wv[k], fw);
#pragma unroll
                    for (int e = 0; e < VEC; ++e) o[e] = rinv * (fg[e] * fw[e] - fx[e] * term2);
                    st_stream16(dr + v, pack16<T>(o));
                }
            }
        }
    }

    // Fold the G group partials in fixed order through the (now idle) slot area, write one row.
    if constexpr (G > 1) {
        constexpr int kRow = TPR * VPT * VEC;
        float* fold = reinterpret_cast<float*>(smem);
        __syncthreads();  // every thread is done reading slots
        if (group > 0) {
#pragma unroll
            for (int k = 0; k < VPT; ++k)
#pragma unroll
                for (int e = 0; e < VEC; ++e) fold[(group - 1) * kRow + (k * VEC + e) * TPR + t] = acc[k][e];
        }
        __syncthreads();
        if (group == 0) {
            for (int q = 0; q < G - 1; ++q)
#pragma unroll
                for (int k = 0; k < VPT; ++k)
#pragma unroll
                    for (int e = 0; e < VEC; ++e) acc[k][e] += fold[q * kRow + (k * VEC + e) * TPR + t];
        }
    }
    if (group == 0) {
        float* out = ws + static_cast<int64_t>(blockIdx.x) * cols;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            if (v < nvec) {
#pragma unroll
                for (int e = 0; e < VEC; e += 4)
                    *reinterpret_cast<float4*>(out + static_cast<int64_t>(v) * VEC + e) =
                        make_float4(acc[k][e], acc[k][e + 1], acc[k][e + 2], acc[k][e + 3]);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag != 0) atomicExch(status, MGR_ERR_DEVICE_TIMEOUT);
}

}  // namespace mgr
