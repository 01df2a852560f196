// RMSNorm forward / backward for sm_100a.
//
// Replaces the six SIMT kernels and six host wrappers of the reference's src/rmsnorm_kernel.cu
// (forward :42-230, backward :235-522, wrappers :529-662). Same arithmetic (fp32 accumulate, one
// rounding on store), different execution plan:
//   * a row lives in registers (16-byte packets), so x (and dy) are read from HBM once per direction
//     -- the reference makes two passes over each row;
//   * CTAs are persistent (grid = SMs x resident CTAs) and keep the weight row in registers, or, where the registers
//     are better spent on rows in flight, in shared memory (rms_bwd_wsm, rms_fwd_reg<.., WSM>);
//   * while a group of threads works on one row, L2 is asked for the row it visits next (prefetch_l2_bulk), by a
//     measured per-case policy (use_prefetch);
//   * dW is accumulated per thread in fp32 registers over all rows a CTA visits, written once as a
//     per-CTA partial row, and summed by a second fixed-order kernel -- no atomics, so dW is
//     bit-reproducible (the reference: atomicAdd at :319-322, half-precision atomics at :421-422).
// Shapes the packet path cannot take (cols not a multiple of the packet width, pointers not 16-byte
// aligned, rows longer than 4096 packets) go to scalar kernels with the same arithmetic.

#include <atomic>

#include "mgr_common.cuh"
#include "rmsnorm_ring.cuh"

namespace mgr {
namespace {

// Set by a kernel whose bounded wait ran out (MGR_ERR_DEVICE_TIMEOUT); read by mgr_device_status().
__device__ int g_rms_status = 0;

// ------------------------------------------------------------------------------------------------
// Packet ("reg") kernels: TPR threads cooperate on one row, each holds VPT 16-byte packets of it.
// A CTA has max(256, TPR) threads and therefore works on G = BLOCK/TPR rows at a time.
// ------------------------------------------------------------------------------------------------

template <int TPR>
struct RegGeom {
    // 256 threads shared by several rows when TPR divides 256, else one row per CTA pass
    static constexpr int kBlock = TPR >= 256 ? TPR : (256 % TPR == 0 ? 256 : TPR);
    static constexpr int kGroups = kBlock / TPR;
    static constexpr int kWarpsPerRow = TPR / 32;
    static constexpr int kWarps = kBlock / 32;
    // resident CTAs per SM the register allocation is held to (forward: 64 registers per thread;
    // backward: 128, which still holds the row packets and the dW partials without spilling)
    static constexpr int kFwdMinBlocks = 1024 / kBlock < 1 ? 1 : 1024 / kBlock;
    static constexpr int kBwdMinBlocks = 512 / kBlock < 1 ? 1 : 512 / kBlock;
};

// Whether a kernel instance carries the code that asks L2 for the next row (prefetch_l2_bulk) at all. The host's
// policy (use_prefetch) never turns it on for the shapes excluded here, and its mere presence costs the kernels
// that are held to 40-64 registers: bf16 hidden 1536 ({192,1}) backward 0.78 with the unused code against 0.93
// without, hidden 5120 ({320,2}) residual-add backward 0.75 against 0.87.
constexpr bool prefetch_compiled(int tpr, int vpt, bool add, bool backward) {
    const int cap = tpr * vpt;
    if (!backward) return cap > 1024;
    if (add) return cap > 128 && !(tpr == 320 && vpt == 2);
    return cap >= 256;
}

// Sum of `v` over the TPR threads that share a row. `red` is a [2][kWarps] shared array used
// alternately (`buf`), which makes one __syncthreads per reduction sufficient.
template <int TPR>
__device__ __forceinline__ float row_sum(float v, float (*red)[RegGeom<TPR>::kWarps], int& buf, int group) {
    v = warp_sum(v);
    if constexpr (RegGeom<TPR>::kWarpsPerRow > 1) {
        constexpr int WPR = RegGeom<TPR>::kWarpsPerRow;
        const int warp = threadIdx.x >> 5;
        if ((threadIdx.x & 31) == 0) red[buf][warp] = v;
        __syncthreads();
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < WPR; ++i) s += red[buf][group * WPR + i];
        buf ^= 1;
        v = s;
    }
    return v;
}

// ADD: the row that is normalised is h = round_T(x + res); h is also written out (the new residual
// stream). h_out may be the buffer of x or of res: a thread reads its packets of a row before it writes them.
// WSM: the weight row is kept in shared memory (one copy per CTA) instead of VPT packets per thread, and the CTA
// meets once, behind its first row's loads, before it reads them. Used by the residual-add form of the shapes whose
// table entry says so (wsm_add): the registers it frees are the ones the second operand would otherwise spill.
template <typename T, int TPR, int VPT, bool ADD = false, bool WSM = false>
// (the warp-per-row shape with four packets per lane is held to 3 CTAs per SM instead of 4: at 64 registers it
// spilled and ran at 0.88 of the copy bandwidth on 2 KB rows; at 77 registers, no spills, 0.95)
__global__ void __launch_bounds__(RegGeom<TPR>::kBlock, (TPR == 32 && VPT == 4) ? 3 : RegGeom<TPR>::kFwdMinBlocks)
rms_fwd_reg(T* __restrict__ y, float* __restrict__ inv_rms, const T* x,
            const T* __restrict__ w, int64_t rows, int cols, float eps, const T* res = nullptr, T* h_out = nullptr, int prefetch = 0) {
    using Geo = RegGeom<TPR>;
    constexpr int VEC = Elem<T>::kVec;
    __shared__ float red[2][Geo::kWarps];
    __shared__ uint4 wsm[WSM ? TPR * VPT : 1];
    int buf = 0;

    const int group = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int nvec = cols / VEC;

    uint4 wv[WSM ? 1 : VPT];
    if constexpr (WSM) {
        for (int v = threadIdx.x; v < TPR * VPT; v += Geo::kBlock)
            wsm[v] = v < nvec ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
    } else {
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            wv[k] = v < nvec ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
        }
    }
    [[maybe_unused]] bool weights_pending = WSM;   // every CTA runs at least one pass of the loop below (grid <= row groups)

    const float inv_cols = 1.0f / static_cast<float>(cols);
    const int64_t ngroups = (rows + Geo::kGroups - 1) / Geo::kGroups;
    [[maybe_unused]] const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
    for (int64_t rg = blockIdx.x; rg < ngroups; rg += gridDim.x) {
        const int64_t r = rg * Geo::kGroups + group;
        const bool live = r < rows;
        if constexpr (prefetch_compiled(TPR, VPT, ADD, false)) {   // the row this group visits next goes on its way into L2
            const int64_t rn = (rg + gridDim.x) * Geo::kGroups + group;
            if (prefetch != 0 && t == 0 && rn < rows) {
                prefetch_l2_bulk(x + rn * static_cast<int64_t>(cols), row_bytes);
                if constexpr (ADD) prefetch_l2_bulk(res + rn * static_cast<int64_t>(cols), row_bytes);
            }
        }
        const uint4* xr = reinterpret_cast<const uint4*>(x + (live ? r : 0) * static_cast<int64_t>(cols));
        uint4 xv[VPT];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            xv[k] = (live && v < nvec) ? ld_stream16(xr + v) : make_uint4(0, 0, 0, 0);
            if constexpr (!WSM) keep_packed(wv[k]);
        }
        if constexpr (ADD) {
            const int64_t off = (live ? r : 0) * static_cast<int64_t>(cols);
            const uint4* rr = reinterpret_cast<const uint4*>(res + off);
            uint4* hr = reinterpret_cast<uint4*>(h_out + off);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                if (live && v < nvec) {
                    const uint4 rv = ld_stream16(rr + v);
                    float f[VEC], g[VEC];
                    unpack16<T>(xv[k], f);
                    unpack16<T>(rv, g);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) f[i] += g[i];
                    xv[k] = pack16<T>(f);
                    st_stream16(hr + v, xv[k]);
                }
            }
        }
        float ss = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            float f[VEC];
            unpack16<T>(xv[k], f);
#pragma unroll
            for (int i = 0; i < VEC; ++i) ss += f[i] * f[i];
        }
        if constexpr (WSM) {
            if (weights_pending) {   // rg is the same for the whole CTA: every thread takes this branch in the same pass
                __syncthreads();
                weights_pending = false;
            }
        }
        ss = row_sum<TPR>(ss, red, buf, group);
        const float inv = 1.0f / sqrtf(ss * inv_cols + eps);
        if (live && t == 0 && inv_rms != nullptr) inv_rms[r] = inv;
        if (live && y != nullptr) {   // y == NULL: only the row scales are wanted (mgr_rms_inv)
            uint4* yr = reinterpret_cast<uint4*>(y + r * static_cast<int64_t>(cols));
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                if (v < nvec) {
                    float f[VEC], g[VEC], o[VEC];
                    unpack16<T>(xv[k], f);
                    if constexpr (WSM) unpack16<T>(wsm[v], g);
                    else unpack16<T>(wv[k], g);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) o[i] = (f[i] * inv) * g[i];
                    st_stream16(yr + v, pack16<T>(o));
                }
            }
        }
    }
}

// Backward. Each thread owns the same VPT*VEC columns for every row its CTA visits, so the dW
// partial sums stay in registers until the CTA is done; the G row groups of a CTA are then folded in
// shared memory (fixed order) and the CTA writes ONE fp32 partial row ws[blockIdx.x, :].
// ADD: dx = round_T(dx_norm + dres), the gradient that arrives along the residual stream folded into the
// same store (one rounding). dx may be the buffer of dres.
template <typename T, int TPR, int VPT, bool ADD = false>
__global__ void __launch_bounds__(RegGeom<TPR>::kBlock, (VPT <= 2 && TPR >= 160) ? (VPT == 1 ? 1536 : 1024) / RegGeom<TPR>::kBlock : RegGeom<TPR>::kBwdMinBlocks)
rms_bwd_reg(T* dx, float* __restrict__ ws, const T* __restrict__ dy, const T* __restrict__ x,
            const T* __restrict__ w, const float* __restrict__ inv_rms, int64_t rows, int cols, const T* dres = nullptr, int prefetch = 0) {
    using Geo = RegGeom<TPR>;
    constexpr int VEC = Elem<T>::kVec;
    constexpr int G = Geo::kGroups;
    constexpr bool kTwoPass = TPR >= 1024;   // 64 registers per thread: the row cannot stay resident
    // Residual gradient fetched together with x and dy (all of a row's loads in flight at once) where the
    // register budget is 128 per thread; elsewhere it is fetched just before the store.
    constexpr bool kEarlyRes = ADD && !kTwoPass;
    __shared__ float red[2][Geo::kWarps];
    __shared__ __align__(16) float fold[G > 1 ? (G - 1) * TPR * VPT * VEC : 4];
    int buf = 0;

    const int group = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int nvec = cols / VEC;

    uint4 wv[VPT];
    float acc[VPT][VEC];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int v = t + k * TPR;
        wv[k] = (!kTwoPass && v < nvec) ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[k][i] = 0.f;
    }

    const float inv_cols = 1.0f / static_cast<float>(cols);
    const int64_t ngroups = (rows + G - 1) / G;
    [[maybe_unused]] const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
    for (int64_t rg = blockIdx.x; rg < ngroups; rg += gridDim.x) {
        const int64_t r = rg * G + group;
        const bool live = r < rows;
        if constexpr (prefetch_compiled(TPR, VPT, ADD, true)) {   // the row this group visits next goes on its way into L2
            const int64_t rn = (rg + gridDim.x) * G + group;
            if (prefetch != 0 && t == 0 && rn < rows) {
                const int64_t offn = rn * static_cast<int64_t>(cols);
                prefetch_l2_bulk(x + offn, row_bytes);
                prefetch_l2_bulk(dy + offn, row_bytes);
                if constexpr (ADD) prefetch_l2_bulk(dres + offn, row_bytes);
            }
        }
        const int64_t off = (live ? r : 0) * static_cast<int64_t>(cols);
        const uint4* xr = reinterpret_cast<const uint4*>(x + off);
        const uint4* gr = reinterpret_cast<const uint4*>(dy + off);
        const float rinv = live ? __ldg(inv_rms + r) : 0.f;
        if constexpr (!kTwoPass) {
            uint4 xv[VPT], gv[VPT];
            uint4 dv[kEarlyRes ? VPT : 1];
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                const bool on = live && v < nvec;
                xv[k] = on ? ld_stream16(xr + v) : make_uint4(0, 0, 0, 0);
                gv[k] = on ? ld_stream16(gr + v) : make_uint4(0, 0, 0, 0);
                if constexpr (kEarlyRes) dv[k] = on ? ld_stream16(reinterpret_cast<const uint4*>(dres + off) + v) : make_uint4(0, 0, 0, 0);
                keep_packed(wv[k]);
            }

            float c = 0.f;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                float fx[VEC], fg[VEC], fw[VEC];
                unpack16<T>(xv[k], fx);
                unpack16<T>(gv[k], fg);
                unpack16<T>(wv[k], fw);
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    c += (fg[i] * fw[i]) * fx[i];
                    acc[k][i] += (fg[i] * fx[i]) * rinv;
                }
            }
            c = row_sum<TPR>(c, red, buf, group);
            const float term2 = c * (rinv * rinv) * inv_cols;

            if (live) {
                uint4* dr = reinterpret_cast<uint4*>(dx + off);
#pragma unroll
                for (int k = 0; k < VPT; ++k) {
                    const int v = t + k * TPR;
                    if (v < nvec) {
                        float fx[VEC], fg[VEC], fw[VEC], o[VEC];
                        unpack16<T>(xv[k], fx);
                        unpack16<T>(gv[k], fg);
                        unpack16<T>(wv[k], fw);
#pragma unroll
                        for (int i = 0; i < VEC; ++i) o[i] = rinv * (fg[i] * fw[i] - fx[i] * term2);
                        if constexpr (ADD) {
                            float fr[VEC];
                            if constexpr (kEarlyRes) unpack16<T>(dv[k], fr);
                            else unpack16<T>(ld_stream16(reinterpret_cast<const uint4*>(dres + off) + v), fr);
#pragma unroll
                            for (int i = 0; i < VEC; ++i) o[i] += fr[i];
                        }
                        st_stream16(dr + v, pack16<T>(o));
                    }
                }
            }
        } else {
            // Rows too long to hold in the registers of 1024 threads next to the dW partials: the row is
            // read twice, packet by packet. The first read comes from HBM and stays cached (plain loads); the
            // second, right behind it, is served by L1/L2, so HBM traffic does not grow.
            float c = 0.f;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                const bool on = live && v < nvec;
                const uint4 px = on ? __ldg(xr + v) : make_uint4(0, 0, 0, 0);
                const uint4 pg = on ? __ldg(gr + v) : make_uint4(0, 0, 0, 0);
                const uint4 pw = v < nvec ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
                float fx[VEC], fg[VEC], fw[VEC];
                unpack16<T>(px, fx);
                unpack16<T>(pg, fg);
                unpack16<T>(pw, fw);
#pragma unroll
                for (int i = 0; i < VEC; ++i) c += (fg[i] * fw[i]) * fx[i];
            }
            c = row_sum<TPR>(c, red, buf, group);
            const float term2 = c * (rinv * rinv) * inv_cols;
            uint4* dr = reinterpret_cast<uint4*>(dx + off);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                if (live && v < nvec) {
                    const uint4 px = ld_stream16(xr + v);
                    const uint4 pg = ld_stream16(gr + v);
                    const uint4 pw = __ldg(reinterpret_cast<const uint4*>(w) + v);   // weights are not kept in registers here
                    float fx[VEC], fg[VEC], fw[VEC], o[VEC];
                    unpack16<T>(px, fx);
                    unpack16<T>(pg, fg);
                    unpack16<T>(pw, fw);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        acc[k][i] += (fg[i] * fx[i]) * rinv;
                        o[i] = rinv * (fg[i] * fw[i] - fx[i] * term2);
                    }
                    if constexpr (ADD) {
                        float fr[VEC];
                        unpack16<T>(ld_stream16(reinterpret_cast<const uint4*>(dres + off) + v), fr);
#pragma unroll
                        for (int i = 0; i < VEC; ++i) o[i] += fr[i];
                    }
                    st_stream16(dr + v, pack16<T>(o));
                }
            }
        }
    }

    // Fold the G groups of this CTA (group 0 adds groups 1..G-1 in order), then one partial row out.
    if constexpr (G > 1) {
        constexpr int kRow = TPR * VPT * VEC;
        if (group > 0) {
#pragma unroll
            for (int k = 0; k < VPT; ++k)
#pragma unroll
                for (int i = 0; i < VEC; ++i) fold[(group - 1) * kRow + (k * VEC + i) * TPR + t] = acc[k][i];
        }
        __syncthreads();
        if (group == 0) {
            for (int gidx = 0; gidx < G - 1; ++gidx)
#pragma unroll
                for (int k = 0; k < VPT; ++k)
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[k][i] += fold[gidx * kRow + (k * VEC + i) * TPR + t];
        }
    }
    if (group == 0) {
        float* out = ws + static_cast<int64_t>(blockIdx.x) * cols;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            if (v < nvec) {
#pragma unroll
                for (int i = 0; i < VEC; i += 4)
                    *reinterpret_cast<float4*>(out + static_cast<int64_t>(v) * VEC + i) =
                        make_float4(acc[k][i], acc[k][i + 1], acc[k][i + 2], acc[k][i + 3]);
            }
        }
    }
}

// Geometry of the backward kernel. One FAT CTA per SM where the register budget allows it: G = kGroups row groups
// of TPR threads each run their own rows independently (they meet only on their own named barrier), and are
// folded in shared memory at the end, so a CTA writes ONE partial row of dW however many rows it had in flight.
// (With one small CTA per row group the same SM wrote 2-6 partial rows; the column sum that follows reads them all.)
// kBudget = resident threads per SM the register allocation is held to: 128 registers per thread in general, 64
// (40) where a thread holds at most two (one) packets of a row.
// (Giving {256,2} 85 registers -- three row groups per SM instead of four, no spills -- was measured too: 0.84 against
// 0.93 for one CTA per row group at bf16 hidden 4096, 24.6 against 22.9 us at 4096 x 4096. Rows in flight matter more.)
constexpr int bwd_budget(int tpr, int vpt) {
    if (tpr == 128 && vpt == 2) return 1024;   // eight groups of 128 threads (rms_bwd_wsm): measured ahead of four, 0.93 against 0.89
    return (vpt <= 2 && tpr >= 160) ? (vpt == 1 ? 1536 : 1024) : 512;
}
constexpr int bwd_groups(int tpr, int vpt) {
    const int budget = bwd_budget(tpr, vpt);
    const int max_block = budget < 1024 ? budget : 1024;
    if (tpr >= max_block) return 1;
    for (int g = max_block / tpr; g >= 1; --g)
        if (budget % (g * tpr) == 0) return g;       // whole CTAs fill the budget
    return max_block / tpr;
}

template <int TPR, int VPT>
struct BwdGeom {
    static constexpr int kGroups = bwd_groups(TPR, VPT);
    static constexpr int kBlock = kGroups * TPR;
    static constexpr int kMinBlocks = bwd_budget(TPR, VPT) / kBlock < 1 ? 1 : bwd_budget(TPR, VPT) / kBlock;
    static constexpr int kWarpsPerRow = TPR / 32;
    static constexpr int kWarps = kBlock / 32;
    static constexpr int kFoldRows = kGroups / 2;    // partial rows parked in shared memory during the fold
};

// Sum of `v` over the TPR threads of one row group. `red` is this group's own [2][TPR/32] slice of shared memory,
// used alternately; the group meets on ITS named barrier (id group + 1), so other groups of the CTA are not held up.
template <int TPR>
__device__ __forceinline__ float group_sum(float v, float* red_all, int& buf, int group) {
    v = warp_sum(v);
    if constexpr (TPR > 32) {
        constexpr int WPR = TPR / 32;
        float* red = red_all + (group * 2 + buf) * WPR;
        if ((threadIdx.x & 31) == 0) red[(threadIdx.x >> 5) - group * WPR] = v;
        asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "n"(TPR) : "memory");
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < WPR; ++i) s += red[i];
        buf ^= 1;
        v = s;
    }
    return v;
}

// Backward. Each thread owns the same VPT*VEC columns for every row its group visits, so the dW partial sums
// stay in registers until the CTA is done; the G groups are then folded pairwise in shared memory (distance 1,
// 2, 4, ...: a fixed tree) and the CTA writes ONE fp32 partial row ws[blockIdx.x, :].
// ADD: dx = round_T(dx_norm + dres), the gradient that arrives along the residual stream folded into the
// same store (one rounding). dx may be the buffer of dres.
template <typename T, int TPR, int VPT, bool ADD = false>
__global__ void __launch_bounds__(BwdGeom<TPR, VPT>::kBlock, BwdGeom<TPR, VPT>::kMinBlocks)
rms_bwd_fat(T* dx, float* __restrict__ ws, const T* __restrict__ dy, const T* __restrict__ x,
            const T* __restrict__ w, const float* __restrict__ inv_rms, int64_t rows, int cols, const T* dres = nullptr, int prefetch = 0) {
    using Geo = BwdGeom<TPR, VPT>;
    constexpr int VEC = Elem<T>::kVec;
    constexpr int G = Geo::kGroups;
    constexpr bool kTwoPass = TPR >= 1024;   // 64 registers per thread: the row cannot stay resident
    // Residual gradient fetched together with x and dy (all of a row's loads in flight at once) where the
    // register budget is 128 per thread; elsewhere it is fetched just before the store.
    constexpr bool kEarlyRes = ADD && !kTwoPass;
    constexpr int kRow = TPR * VPT * VEC;
    __shared__ float red_all[2 * Geo::kWarps];
    __shared__ __align__(16) float fold[Geo::kFoldRows > 0 ? Geo::kFoldRows * kRow : 4];
    int buf = 0;

    const int group = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int nvec = cols / VEC;
    float* const red = red_all;

    uint4 wv[VPT];
    float acc[VPT][VEC];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int v = t + k * TPR;
        wv[k] = (!kTwoPass && v < nvec) ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[k][i] = 0.f;
    }

    const float inv_cols = 1.0f / static_cast<float>(cols);
    // Rows are dealt G at a time to the CTAs round robin, one to each group; every thread of a group sees the same
    // rows, so the early exit below is taken by whole groups. (Written with the row-group counter as the loop
    // variable: the form that counts rows directly costs the half-precision kernels 50-80 bytes more in spills.)
    const int64_t ngroups = (rows + G - 1) / G;
    [[maybe_unused]] const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
    for (int64_t rg = blockIdx.x; rg < ngroups; rg += gridDim.x) {
        const int64_t r = rg * G + group;
        if (r >= rows) break;
        if constexpr (prefetch_compiled(TPR, VPT, ADD, true)) {   // the row this group visits next goes on its way into L2
            const int64_t rn = (rg + gridDim.x) * G + group;
            if (prefetch != 0 && t == 0 && rn < rows) {
                const int64_t offn = rn * static_cast<int64_t>(cols);
                prefetch_l2_bulk(x + offn, row_bytes);
                prefetch_l2_bulk(dy + offn, row_bytes);
                if constexpr (ADD) prefetch_l2_bulk(dres + offn, row_bytes);
            }
        }
        const int64_t off = r * static_cast<int64_t>(cols);
        const uint4* xr = reinterpret_cast<const uint4*>(x + off);
        const uint4* gr = reinterpret_cast<const uint4*>(dy + off);
        const float rinv = __ldg(inv_rms + r);
        if constexpr (!kTwoPass) {
            uint4 xv[VPT], gv[VPT];
            uint4 dv[kEarlyRes ? VPT : 1];
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                const bool on = v < nvec;
                xv[k] = on ? ld_stream16(xr + v) : make_uint4(0, 0, 0, 0);
                gv[k] = on ? ld_stream16(gr + v) : make_uint4(0, 0, 0, 0);
                if constexpr (kEarlyRes) dv[k] = on ? ld_stream16(reinterpret_cast<const uint4*>(dres + off) + v) : make_uint4(0, 0, 0, 0);
                keep_packed(wv[k]);
            }

            float c = 0.f;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                float fx[VEC], fg[VEC], fw[VEC];
                unpack16<T>(xv[k], fx);
                unpack16<T>(gv[k], fg);
                unpack16<T>(wv[k], fw);
#pragma unroll
                for (int i = 0; i < VEC; ++i) {
                    c += (fg[i] * fw[i]) * fx[i];
                    acc[k][i] += (fg[i] * fx[i]) * rinv;
                }
            }
            c = group_sum<TPR>(c, red, buf, group);
            const float term2 = c * (rinv * rinv) * inv_cols;

            uint4* dr = reinterpret_cast<uint4*>(dx + off);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                if (v < nvec) {
                    float fx[VEC], fg[VEC], fw[VEC], o[VEC];
                    unpack16<T>(xv[k], fx);
                    unpack16<T>(gv[k], fg);
                    unpack16<T>(wv[k], fw);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) o[i] = rinv * (fg[i] * fw[i] - fx[i] * term2);
                    if constexpr (ADD) {
                        float fr[VEC];
                        if constexpr (kEarlyRes) unpack16<T>(dv[k], fr);
                        else unpack16<T>(ld_stream16(reinterpret_cast<const uint4*>(dres + off) + v), fr);
#pragma unroll
                        for (int i = 0; i < VEC; ++i) o[i] += fr[i];
                    }
                    st_stream16(dr + v, pack16<T>(o));
                }
            }
        } else {
            // Rows too long to hold in the registers of 1024 threads next to the dW partials: the row is
            // read twice, packet by packet. The first read comes from HBM and stays cached (plain loads); the
            // second, right behind it, is served by L1/L2, so HBM traffic does not grow.
            float c = 0.f;
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                const bool on = v < nvec;
                const uint4 px = on ? __ldg(xr + v) : make_uint4(0, 0, 0, 0);
                const uint4 pg = on ? __ldg(gr + v) : make_uint4(0, 0, 0, 0);
                const uint4 pw = on ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
                float fx[VEC], fg[VEC], fw[VEC];
                unpack16<T>(px, fx);
                unpack16<T>(pg, fg);
                unpack16<T>(pw, fw);
#pragma unroll
                for (int i = 0; i < VEC; ++i) c += (fg[i] * fw[i]) * fx[i];
            }
            c = group_sum<TPR>(c, red, buf, group);
            const float term2 = c * (rinv * rinv) * inv_cols;
            uint4* dr = reinterpret_cast<uint4*>(dx + off);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                if (v < nvec) {
                    const uint4 px = ld_stream16(xr + v);
                    const uint4 pg = ld_stream16(gr + v);
                    const uint4 pw = __ldg(reinterpret_cast<const uint4*>(w) + v);   // weights are not kept in registers here
                    float fx[VEC], fg[VEC], fw[VEC], o[VEC];
                    unpack16<T>(px, fx);
                    unpack16<T>(pg, fg);
                    unpack16<T>(pw, fw);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) {
                        acc[k][i] += (fg[i] * fx[i]) * rinv;
                        o[i] = rinv * (fg[i] * fw[i] - fx[i] * term2);
                    }
                    if constexpr (ADD) {
                        float fr[VEC];
                        unpack16<T>(ld_stream16(reinterpret_cast<const uint4*>(dres + off) + v), fr);
#pragma unroll
                        for (int i = 0; i < VEC; ++i) o[i] += fr[i];
                    }
                    st_stream16(dr + v, pack16<T>(o));
                }
            }
        }
    }

    // Fold the G groups of this CTA: at distance d = 1, 2, 4, ... group g with g % 2d == d hands its sums to group
    // g - d through shared memory. A fixed tree, so the CTA's partial row does not depend on timing.
    if constexpr (G > 1) {
#pragma unroll
        for (int d = 1; d < G; d <<= 1) {
            const int pos = group & (2 * d - 1);
            float* slot = fold + (group / (2 * d)) * kRow;
            if (pos == d) {
#pragma unroll
                for (int k = 0; k < VPT; ++k)
#pragma unroll
                    for (int i = 0; i < VEC; ++i) slot[(k * VEC + i) * TPR + t] = acc[k][i];
            }
            __syncthreads();
            if (pos == 0 && group + d < G) {
#pragma unroll
                for (int k = 0; k < VPT; ++k)
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[k][i] += slot[(k * VEC + i) * TPR + t];
            }
            __syncthreads();
        }
    }
    if (group == 0) {
        float* out = ws + static_cast<int64_t>(blockIdx.x) * cols;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            if (v < nvec) {
#pragma unroll
                for (int i = 0; i < VEC; i += 4)
                    *reinterpret_cast<float4*>(out + static_cast<int64_t>(v) * VEC + i) =
                        make_float4(acc[k][i], acc[k][i + 1], acc[k][i + 2], acc[k][i + 3]);
            }
        }
    }
}

// Backward, fat CTA with the weight row in shared memory (one copy per CTA, read by every group) instead of VPT
// packets per thread. The registers this frees are what lets four groups of {128,4} (eight of {128,2}) run without
// spills at one CTA per SM, so the kernel writes 148 partial rows where one CTA per row group wrote 592-888, and the
// column sum behind it reads a quarter of the bytes. The fill is ordered behind the first row's loads: a thread
// requests its first packets, then the CTA meets once, so the weights cost no round trip of their own. After the row
// loop the same shared memory is the fold buffer.
// Measured on B200 (bf16, fraction of the copy bandwidth, backward call with its column sum, this form against one
// CTA per row group): hidden 4096 at 65 536 / 16 384 / 8192 / 4096 rows 0.95 / 0.86 / 0.79 / 0.68 against
// 0.92 / 0.84 / 0.76 / 0.64; hidden 2048 at 262 144 / 8192 rows 0.96 / 0.69 against 0.93 / 0.67.
// The row loop counts rows in 32 bits and fetches the row scale behind the packets: both forms were timed, and the
// 64-bit row-group counter of rms_bwd_fat costs this kernel 2.5 % and the scale fetched first another 0.7 %.
// The host sends problems of 2^31 rows or more to the other kernels.
template <typename T, int TPR, int VPT, bool ADD = false>
__global__ void __launch_bounds__(BwdGeom<TPR, VPT>::kBlock, BwdGeom<TPR, VPT>::kMinBlocks)
// (dx carries __restrict__ although the residual-add form allows dx == dres: a thread reads its packets of a row
// before it writes them and no other thread touches them, so no reordering the qualifier permits can change a value)
rms_bwd_wsm(T* __restrict__ dx, float* __restrict__ ws, const T* __restrict__ dy, const T* __restrict__ x,
            const T* __restrict__ w, const float* __restrict__ inv_rms, int rows, int cols, const T* dres = nullptr, int prefetch = 0) {
    using Geo = BwdGeom<TPR, VPT>;
    constexpr int VEC = Elem<T>::kVec;
    constexpr int G = Geo::kGroups;
    constexpr int kRow = TPR * VPT * VEC;
    constexpr int kBlock = G * TPR;
    static_assert(TPR < 1024, "rows that need the two-pass form keep their weights in global memory");
    __shared__ float red_all[2 * (kBlock / 32)];
    constexpr int kFoldBytes = G / 2 > 0 ? (G / 2) * kRow * 4 : 16;
    constexpr int kWeightBytes = TPR * VPT * 16;
    __shared__ __align__(16) unsigned char pool[kFoldBytes > kWeightBytes ? kFoldBytes : kWeightBytes];   // weights during the row loop, fold buffer after it
    float* fold = reinterpret_cast<float*>(pool);
    uint4* wsm = reinterpret_cast<uint4*>(pool);
    int buf = 0;
    const int group = threadIdx.x / TPR;
    const int t = threadIdx.x % TPR;
    const int nvec = cols / VEC;
    float acc[VPT][VEC];
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[k][i] = 0.f;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    int r = blockIdx.x * G + group;
    uint4 xv[VPT], gv[VPT];
    [[maybe_unused]] uint4 dv[ADD ? VPT : 1];
    float rinv = 0.f;
    // every load of a row, issued back to back; the row scale goes last (timed: 0.7 % ahead of first)
    auto load = [&](int row) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<int64_t>(row) * cols);
        const uint4* gr = reinterpret_cast<const uint4*>(dy + static_cast<int64_t>(row) * cols);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            const bool on = v < nvec;
            xv[k] = on ? ld_stream16(xr + v) : make_uint4(0, 0, 0, 0);
            gv[k] = on ? ld_stream16(gr + v) : make_uint4(0, 0, 0, 0);
        }
        if constexpr (ADD) {
            const uint4* rr = reinterpret_cast<const uint4*>(dres + static_cast<int64_t>(row) * cols);
#pragma unroll
            for (int k = 0; k < VPT; ++k) {
                const int v = t + k * TPR;
                dv[k] = v < nvec ? ld_stream16(rr + v) : make_uint4(0, 0, 0, 0);
            }
        }
        rinv = __ldg(inv_rms + row);
    };
    for (int v = threadIdx.x; v < TPR * VPT; v += kBlock)
        wsm[v] = v < nvec ? __ldg(reinterpret_cast<const uint4*>(w) + v) : make_uint4(0, 0, 0, 0);
    const int stride = gridDim.x * G;
    bool weights_pending = true;   // every thread meets the CTA exactly once, behind its first row's loads
    [[maybe_unused]] const uint32_t row_bytes = static_cast<uint32_t>(cols) * sizeof(T);
    for (; r < rows; r += stride) {
        if constexpr (prefetch_compiled(TPR, VPT, ADD, true)) {   // the row this group visits next goes on its way into L2
            if (prefetch != 0 && t == 0 && r + stride < rows) {
                const int64_t offn = static_cast<int64_t>(r + stride) * cols;
                prefetch_l2_bulk(x + offn, row_bytes);
                prefetch_l2_bulk(dy + offn, row_bytes);
                if constexpr (ADD) prefetch_l2_bulk(dres + offn, row_bytes);
            }
        }
        load(r);
        if (weights_pending) { __syncthreads(); weights_pending = false; }
        float c = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            float fx[VEC], fg[VEC], fw[VEC];
            unpack16<T>(xv[k], fx);
            unpack16<T>(gv[k], fg);
            unpack16<T>(wsm[t + k * TPR], fw);
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
                c += (fg[i] * fw[i]) * fx[i];
                acc[k][i] += (fg[i] * fx[i]) * rinv;
            }
        }
        c = group_sum<TPR>(c, red_all, buf, group);
        const float term2 = c * (rinv * rinv) * inv_cols;
        uint4* dr = reinterpret_cast<uint4*>(dx + static_cast<int64_t>(r) * cols);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            if (v < nvec) {
                float fx[VEC], fg[VEC], fw[VEC], o[VEC];
                unpack16<T>(xv[k], fx);
                unpack16<T>(gv[k], fg);
                unpack16<T>(wsm[v], fw);
#pragma unroll
                for (int i = 0; i < VEC; ++i) o[i] = rinv * (fg[i] * fw[i] - fx[i] * term2);
                if constexpr (ADD) {
                    float fr[VEC];
                    unpack16<T>(dv[k], fr);
#pragma unroll
                    for (int i = 0; i < VEC; ++i) o[i] += fr[i];
                }
                st_stream16(dr + v, pack16<T>(o));
            }
        }
    }
    if (weights_pending) __syncthreads();   // a group that was dealt no row still owes the CTA its one meeting

    // Fold the G groups (the fixed tree of rms_bwd_fat), then one partial row out.
    if constexpr (G > 1) {
        __syncthreads();   // every group has read its last weights: the pool becomes the fold buffer
#pragma unroll
        for (int d = 1; d < G; d <<= 1) {
            const int pos = group & (2 * d - 1);
            float* slot = fold + (group / (2 * d)) * kRow;
            if (pos == d) {
#pragma unroll
                for (int k = 0; k < VPT; ++k)
#pragma unroll
                    for (int i = 0; i < VEC; ++i) slot[(k * VEC + i) * TPR + t] = acc[k][i];
            }
            __syncthreads();
            if (pos == 0 && group + d < G) {
#pragma unroll
                for (int k = 0; k < VPT; ++k)
#pragma unroll
                    for (int i = 0; i < VEC; ++i) acc[k][i] += slot[(k * VEC + i) * TPR + t];
            }
            __syncthreads();
        }
    }
    if (group == 0) {
        float* out = ws + static_cast<int64_t>(blockIdx.x) * cols;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int v = t + k * TPR;
            if (v < nvec) {
#pragma unroll
                for (int i = 0; i < VEC; i += 4)
                    *reinterpret_cast<float4*>(out + static_cast<int64_t>(v) * VEC + i) =
                        make_float4(acc[k][i], acc[k][i + 1], acc[k][i + 2], acc[k][i + 3]);
            }
        }
    }
}

// dw[j] = sum_{p<P} ws[p, j] for cols % 4 == 0. A CTA of 1024 threads takes 8 packets of four columns (128 bytes of
// every partial row) and cuts the P rows into 128 slices, so that a thread loads only ceil(P / 128) packets, all at
// once: the sum is one round trip to L2 deep instead of a chain of them. Fixed order: a thread adds its rows in
// increasing p; the four slices of a warp are folded by shuffles (distance 1, then 2); the 32 warp sums of a
// column packet are added in increasing warp order by one thread. One rounding to T at the end.
template <typename T>
__global__ void __launch_bounds__(1024)
rms_dw_reduce4(T* __restrict__ dw, float* __restrict__ dw_f32, const float* __restrict__ ws, int P, int cols) {
    __shared__ float4 part[32][8];
    asm volatile("griddepcontrol.wait;" ::: "memory");   // see rms_dw_reduce
    const int c4 = cols >> 2;
    const int lane_col = threadIdx.x & 7;
    const int slice = threadIdx.x >> 3;                  // 0..127
    const int col = static_cast<int>(blockIdx.x) * 8 + lane_col;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (col < c4) {
        const float4* src = reinterpret_cast<const float4*>(ws) + col;
        int p = slice;
        for (; p + 128 < P; p += 256) {
            const float4 v0 = __ldcg(src + static_cast<int64_t>(p) * c4);
            const float4 v1 = __ldcg(src + static_cast<int64_t>(p + 128) * c4);
            a.x += v0.x, a.y += v0.y, a.z += v0.z, a.w += v0.w;
            a.x += v1.x, a.y += v1.y, a.z += v1.z, a.w += v1.w;
        }
        if (p < P) {
            const float4 v0 = __ldcg(src + static_cast<int64_t>(p) * c4);
            a.x += v0.x, a.y += v0.y, a.z += v0.z, a.w += v0.w;
        }
    }
#pragma unroll
    for (int m = 8; m <= 16; m <<= 1) {                   // lanes 8 apart hold neighbouring slices of the same packet
        a.x += __shfl_xor_sync(0xffffffffu, a.x, m);
        a.y += __shfl_xor_sync(0xffffffffu, a.y, m);
        a.z += __shfl_xor_sync(0xffffffffu, a.z, m);
        a.w += __shfl_xor_sync(0xffffffffu, a.w, m);
    }
    if ((threadIdx.x & 31) < 8) part[threadIdx.x >> 5][lane_col] = a;
    __syncthreads();
    if (threadIdx.x < 8 && col < c4) {
        float4 s = part[0][threadIdx.x];
#pragma unroll
        for (int i = 1; i < 32; ++i) {
            const float4 v = part[i][threadIdx.x];
            s.x += v.x, s.y += v.y, s.z += v.z, s.w += v.w;
        }
        const int64_t j = static_cast<int64_t>(col) * 4;
        if (dw != nullptr) {
            dw[j] = from_f32<T>(s.x);
            dw[j + 1] = from_f32<T>(s.y);
            dw[j + 2] = from_f32<T>(s.z);
            dw[j + 3] = from_f32<T>(s.w);
        }
        if (dw_f32 != nullptr) {
            dw_f32[j] = s.x;
            dw_f32[j + 1] = s.y;
            dw_f32[j + 2] = s.z;
            dw_f32[j + 3] = s.w;
        }
    }
}

// dw[j] = sum_{p<P} ws[p, j], summed in a fixed order: each of the 32 slices adds its rows
// p = slice, slice+32, ... in increasing p, then the 32 slice sums are added in increasing slice.
// One rounding to T at the end; the unrounded fp32 sum goes to dw_f32 when asked for.
template <typename T>
__global__ void __launch_bounds__(1024)
rms_dw_reduce(T* __restrict__ dw, float* __restrict__ dw_f32, const float* __restrict__ ws, int P, int cols) {
    __shared__ float part[32][33];
    // Launched as a programmatic dependent of the backward kernel: its CTAs may be scheduled while that
    // kernel drains; this wait returns once the backward kernel has completed and its partial rows are
    // visible. (A no-op when the launch carries no such dependency.)
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int col = blockIdx.x * 32 + threadIdx.x;
    float a = 0.f;
    if (col < cols) {
        int p = threadIdx.y;
        for (; p + 96 < P; p += 128) {
            const float v0 = ws[static_cast<int64_t>(p) * cols + col];
            const float v1 = ws[static_cast<int64_t>(p + 32) * cols + col];
            const float v2 = ws[static_cast<int64_t>(p + 64) * cols + col];
            const float v3 = ws[static_cast<int64_t>(p + 96) * cols + col];
            a += v0;
            a += v1;
            a += v2;
            a += v3;
        }
        for (; p < P; p += 32) a += ws[static_cast<int64_t>(p) * cols + col];
    }
    part[threadIdx.y][threadIdx.x] = a;
    __syncthreads();
    if (threadIdx.y == 0 && col < cols) {
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) s += part[i][threadIdx.x];
        if (dw != nullptr) dw[col] = from_f32<T>(s);
        if (dw_f32 != nullptr) dw_f32[col] = s;
    }
}

// ------------------------------------------------------------------------------------------------
// Scalar kernels: any cols >= 1, any element-aligned pointers. One CTA per row, two passes.
// ------------------------------------------------------------------------------------------------

__device__ __forceinline__ float block_sum_256(float v, float* red /* [8] */) {
    v = warp_sum(v);
    __syncthreads();  // protects `red` from the previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += red[i];
    return s;
}

template <typename T, bool ADD = false>
__global__ void __launch_bounds__(256)
rms_fwd_scalar(T* __restrict__ y, float* __restrict__ inv_rms, const T* x,
               const T* __restrict__ w, int64_t rows, int64_t cols, float eps, const T* res = nullptr, T* h_out = nullptr) {
    __shared__ float red[8];
    const float inv_cols = 1.0f / static_cast<float>(cols);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T* xr = ADD ? h_out + r * cols : x + r * cols;
        T* yr = y + r * cols;
        float ss = 0.f;
        for (int64_t j = threadIdx.x; j < cols; j += 256) {
            if constexpr (ADD) h_out[r * cols + j] = from_f32<T>(to_f32(x[r * cols + j]) + to_f32(res[r * cols + j]));
            const float f = to_f32(xr[j]);   // with ADD: the element this thread has just written
            ss += f * f;
        }
        ss = block_sum_256(ss, red);
        const float inv = 1.0f / sqrtf(ss * inv_cols + eps);
        if (threadIdx.x == 0 && inv_rms != nullptr) inv_rms[r] = inv;
        if (y == nullptr) continue;   // only the row scales are wanted
        for (int64_t j = threadIdx.x; j < cols; j += 256)
            yr[j] = from_f32<T>((to_f32(xr[j]) * inv) * to_f32(w[j]));
    }
}

template <typename T, bool ADD = false>
__global__ void __launch_bounds__(256)
rms_bwd_dx_scalar(T* dx, const T* __restrict__ dy, const T* __restrict__ x,
                  const T* __restrict__ w, const float* __restrict__ inv_rms, int64_t rows, int64_t cols, const T* dres = nullptr) {
    __shared__ float red[8];
    const float inv_cols = 1.0f / static_cast<float>(cols);
    for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T* xr = x + r * cols;
        const T* gr = dy + r * cols;
        T* dr = dx + r * cols;
        const float rinv = inv_rms[r];
        float c = 0.f;
        for (int64_t j = threadIdx.x; j < cols; j += 256) c += (to_f32(gr[j]) * to_f32(w[j])) * to_f32(xr[j]);
        c = block_sum_256(c, red);
        const float term2 = c * (rinv * rinv) * inv_cols;
        for (int64_t j = threadIdx.x; j < cols; j += 256) {
            float o = rinv * (to_f32(gr[j]) * to_f32(w[j]) - to_f32(xr[j]) * term2);
            if constexpr (ADD) o += to_f32(dres[r * cols + j]);
            dr[j] = from_f32<T>(o);
        }
    }
}

// Partial column sums: slice s = blockIdx.y adds rows s, s+S, s+2S, ... (increasing) of column j.
template <typename T>
__global__ void __launch_bounds__(128)
rms_bwd_dw_scalar(float* __restrict__ ws, const T* __restrict__ dy, const T* __restrict__ x,
                  const float* __restrict__ inv_rms, int64_t rows, int64_t cols) {
    const int64_t j = static_cast<int64_t>(blockIdx.x) * 128 + threadIdx.x;
    if (j >= cols) return;
    float a = 0.f;
    for (int64_t r = blockIdx.y; r < rows; r += gridDim.y)
        a += (to_f32(dy[r * cols + j]) * to_f32(x[r * cols + j])) * inv_rms[r];
    ws[static_cast<int64_t>(blockIdx.y) * cols + j] = a;
}

// ------------------------------------------------------------------------------------------------
// Host: plan selection and launches
// ------------------------------------------------------------------------------------------------

struct RegShape {
    int tpr, vpt;
    bool fwd_ok, bwd_ok;   // fitted shapes only: whether the forward / the backward may pick it (from measurements)
    bool fat_bwd;          // backward: one fat CTA per SM (rms_bwd_fat) instead of one CTA per row group (rms_bwd_reg)
    bool fat_wsm = false;  // ... in the form that keeps the weight row in shared memory (rms_bwd_wsm), at every row count
    bool wsm_add = false;  // the residual-add kernels alone take the shared-memory-weights forms (backward: rms_bwd_wsm;
                           // forward: rms_fwd_reg with WSM): their third operand costs the plain forms spills. Measured
                           // on B200 (backward, fraction of the copy bandwidth, bf16): {256,4} at hidden 8192 0.98 against
                           // 0.91, {384,2} at hidden 6144 0.98 against 0.91; without the residual the plain forms stay
                           // ahead there (0.925 against 0.915), and the other shapes lose either way.
    bool fwd_wsm = false;  // the plain forward of a 16-bit type takes the shared-memory-weights form too, when there are rows enough
};
// Indices 8-10 are alternatives to {128,4}, {256,4} and {128,2} with one row per CTA pass; only the backward
// picks them (bwd_shape_for), the size-ordered search of reg_shape_for never reaches them.
// From kFirstFitted on: shapes whose capacity TPR*VPT fits hidden sizes that are not powers of two (bf16: 2560,
// 1536, 3072, 5120, 6144, 7168). A row of 640 packets in the {256,4} shape leaves 3 of every 8 packet slots, and the
// loads that would fill them, empty. Measured on B200 (bf16, 2^28 elements, fraction of the copy bandwidth, fitted
// against the power-of-two choice):
//   backward: 1536: 0.91 / 0.80   2560: 0.92 / 0.76   3072: 0.91 / 0.83   5120: 0.89 / 0.74   6144: 0.84 / 0.80   7168: 0.87 / 0.86
//   forward : 1536: 0.89 / 0.73   2560: 0.88 / 0.80   3072: 0.89 / 0.87 (fp32: 0.90 / 0.96)
//             5120: 0.77 / 0.87   6144: 0.82 / 0.93   7168: 0.70 / 0.97  -- one row per pass of a 320-448 thread
//             CTA with two packets per thread keeps too little in flight per barrier; the forward stays with {256,4}
// ({768,2} for 12288 lost both ways, 0.53 / 0.85 and 0.70 / 0.73, and is not built.)
// fat_bwd, measured on B200 (2^29 elements, fraction of the copy bandwidth, fat / thin): warp-per-row shapes (16
// independent warps in one CTA, no barrier in the row loop) 0.98 / 0.90 at bf16 hidden 1024 and 0.98 / 0.80 at fp32
// hidden 128, equal elsewhere; {512,4} 0.84 / 0.82 at bf16 hidden 16384, 0.96 / 0.95 at fp32 hidden 8192. The other
// shapes keep one CTA per row group: their fat forms need a few registers more than the 64 (128) they are held to
// and lose more to spills than the fewer partial rows give back (bf16 hidden 4096: 0.67 / 0.90; 8192: 0.88 / 0.93;
// fp32 hidden 1024: 0.95 / 1.00).
constexpr RegShape kRegShapes[] = {{32, 1, true, true, true},     {32, 2, true, true, true},    {32, 4, true, true, true},
                                   {128, 2, true, true, true, true, false, true}, {128, 4, true, true, true, true, false, true}, {256, 4, true, true, false, false, true},
                                   {512, 4, true, true, true},    {1024, 4, true, true, false}, {256, 2, true, true, false},
                                   {512, 2, true, true, false},   {256, 1, true, true, false},  {160, 2, false, true, false},
                                   {192, 1, true, true, false},   {192, 2, false, true, false}, {320, 2, false, true, false},
                                   {384, 2, false, true, false, false, true},  {448, 2, false, true, false},
                                   // forward only: four packets per thread (as {128,4}, the best forward shape of its size
                                   // class) at 96 / 160 / 192 threads per row, for rows of 257-384 / 513-640 / 641-768 packets.
                                   // Measured (bf16, 2^29 elements, fraction of the copy bandwidth): hidden 2560 0.98 against 0.87
                                   // for {160,2}; 3072 0.95 against 0.86 for {128,4}; 5120 0.99 against 0.85 for {256,4}.
                                   {96, 4, true, false, false},   {160, 4, true, false, false}, {192, 4, true, false, false},
                                   // rows of 1025-1536 packets (hidden 12288 in bf16): {512,4} leaves a quarter of its slots empty
                                   {384, 4, true, true, true}};
constexpr int kNumRegShapes = sizeof(kRegShapes) / sizeof(kRegShapes[0]);
constexpr int kFirstFitted = 11;
constexpr int kScalarDwSlices = 64;

constexpr int64_t shape_capacity(int i) { return static_cast<int64_t>(kRegShapes[i].tpr) * kRegShapes[i].vpt; }

// MGR_RMSNORM_FWD_SHAPE / MGR_RMSNORM_BWD_SHAPE=<index into kRegShapes> pin the packet shape when it can hold the
// row (measurement aid). Returns -1 when unset or unusable.
int pinned_shape(int i, int64_t nvec) {
    return (i >= 0 && i < kNumRegShapes && nvec <= shape_capacity(i)) ? i : -1;
}

// The fitted shape with the least capacity that still holds the row, if it is tighter than `base` (the choice of
// the power-of-two shapes); else `base`.
constexpr int tighter_fitted(int64_t nvec, int base, bool backward) {
    int best = base;
    for (int i = kFirstFitted; i < kNumRegShapes; ++i) {
        if (!(backward ? kRegShapes[i].bwd_ok : kRegShapes[i].fwd_ok) || nvec > shape_capacity(i)) continue;
        if (best < 0 || shape_capacity(i) < shape_capacity(best)) best = i;
    }
    return best;
}

// Index of the first power-of-two packet shape (table order = capacity order) that holds a row of `nvec` packets, or -1.
constexpr int reg_shape_for(int64_t nvec) {
    for (int i = 0; i < kFirstFitted; ++i)
        if (nvec <= shape_capacity(i)) return i;
    return -1;
}
constexpr int default_fwd_shape(int64_t nvec) { return tighter_fitted(nvec, reg_shape_for(nvec), false); }
// add16: the residual-add backward of a 16-bit type, whose third operand costs {128,2} in eight groups its register
// budget (112 bytes of spills at 64 registers: 0.79 against 0.92 for {256,1}, bf16 hidden 2048); it keeps {256,1}.
constexpr int default_bwd_shape(int64_t nvec, bool add16 = false) {
    // Measured on B200 (bf16, 2^29 elements, fraction of the copy bandwidth): rows of 257-512 packets run at
    // 0.92 with {256,2} (one row per pass, 4 CTAs per SM) against 0.86 with {128,4}; rows of 513-1024 packets
    // are better left with {256,4} (0.92 against 0.89 for {512,2}).
    // Rows of 129-256 packets: 0.93 with {256,1} against 0.76 with {128,2} (and 0.84 for the ring kernel).
    // Both have since given way to fat CTAs with the weights in shared memory (rms_bwd_wsm): {128,4} in four groups
    // for rows of 257-512 packets (0.95 against 0.92) and {128,2} in eight groups for 129-256 packets (0.96 against
    // 0.93), which is what the size-ordered search returns for them. MGR_RMSNORM_BWD_SHAPE=8 / 10 bring the earlier
    // choices back for comparison.
    int base = reg_shape_for(nvec);
    if (add16 && nvec > 128 && nvec <= 256) base = 10;
    // ... and where the fitted shapes lose to the shared-memory-weights form of the power-of-two shape above them
    // (residual-add backward, bf16, fraction of the copy bandwidth): hidden 2560 0.87 with {128,4} against 0.83 with
    // {160,2}; 3072 0.94 against 0.84 with {192,2}; 7168 0.96 with {256,4} against 0.93 with {448,2}. (Not at 5120:
    // 0.83 against 0.87 with {320,2}.)
    if (add16 && ((nvec > 256 && nvec <= 384) || (nvec > 768 && nvec <= 896))) return base;
    return tighter_fitted(nvec, base, true);
}
// Checked at compile time: every row of up to 4096 packets gets a shape that holds it (forward and backward),
// longer rows get none (they take the scalar kernels), and every shape is launchable: whole warps per row, at
// most 1024 threads, and the backward's fold buffer within the static shared-memory limit.
constexpr bool shape_tables_ok() {
    for (int i = 0; i < kNumRegShapes; ++i) {
        const int tpr = kRegShapes[i].tpr, vpt = kRegShapes[i].vpt;
        const int block = tpr >= 256 ? tpr : (256 % tpr == 0 ? 256 : tpr);
        if (tpr % 32 != 0 || block > 1024 || block % tpr != 0 || vpt < 1 || vpt > 4) return false;
        const int bg = bwd_groups(tpr, vpt);
        if (bg * tpr > 1024 || bg < 1 || (tpr > 32 && bg > 15)) return false;                       // a launchable CTA; named barriers 1..15
        if (static_cast<int64_t>(bg / 2) * tpr * vpt * 8 * 4 > 44 * 1024) return false;              // the fold buffer (static shared memory)
    }
    for (int64_t nvec = 1; nvec <= 4096; ++nvec) {
        const int f = default_fwd_shape(nvec), b = default_bwd_shape(nvec), ba = default_bwd_shape(nvec, true);
        if (f < 0 || b < 0 || ba < 0 || shape_capacity(f) < nvec || shape_capacity(b) < nvec || shape_capacity(ba) < nvec) return false;
    }
    return default_fwd_shape(4097) < 0 && default_bwd_shape(4097) < 0;
}
static_assert(shape_tables_ok(), "a row length has no packet shape, or a shape cannot be launched");

int fwd_shape_for(int64_t nvec) {
    const int pinned = pinned_shape(overrides().fwd_shape, nvec);
    return pinned >= 0 ? pinned : default_fwd_shape(nvec);
}
int bwd_shape_for(int64_t nvec, bool add16 = false) {
    const int pinned = pinned_shape(overrides().bwd_shape, nvec);
    return pinned >= 0 ? pinned : default_bwd_shape(nvec, add16);
}

// Whether a packet kernel asks L2 for its next row while it works on the current one (prefetch_l2_bulk). From
// measurements on B200, 2^28 elements, fraction of the copy bandwidth with / without (MGR_RMSNORM_PREFETCH=0|1 pins it):
//   backward, bf16: hidden 2048 0.95 / 0.94, 2560 0.98 / 0.93, 3072 0.99 / 0.93, 4096 0.98 / 0.96, 5120 0.99 / 0.89,
//     6144 0.98 / 0.85, 7168 1.02 / 0.88, 8192 1.00 / 0.93, 12 288 0.91 / 0.75, 16 384 0.95 / 0.84 (the ring: 0.87),
//     32 768 0.95 / 0.71 -- but hidden 1024 0.92 / 1.00 and 1536 0.77 / 0.93: rows of 2-3 KB mean many small requests;
//   backward, fp32: hidden 4096 1.03 / 0.97, 8192 1.05 / 0.98 -- but 1024 0.96 / 1.05 and 2048 0.98 / 1.01;
//   residual-add backward, bf16: hidden 1536 1.05 / 0.93, 2048 1.04 / 0.92, 2560-4096 0.99-1.03 / 0.87-0.99, 6144-12 288
//     1.04-1.07 / 0.96-0.99, 32 768 0.82 / 0.73 -- but 5120 ({320,2}, one CTA per row) 0.71 / 0.87; fp32 4096 1.01 / 1.06;
//   forward: already at the copy rate without it and slower with (bf16 hidden 4096 0.91 / 1.00, 8192 0.92 / 0.99),
//     except for rows beyond 16 KB: hidden 12 288 0.98 / 0.86, 16 384 0.94 / 0.94, 32 768 0.99 / 0.80.
// (The shapes for which this never says yes do not carry the code at all: prefetch_compiled.)
bool use_prefetch(bool backward, bool add, size_t elem, int64_t nvec) {
    const int pinned = overrides().prefetch;
    if (pinned >= 0) return pinned != 0;
    if (!backward) return nvec > 1024;
    if (elem == 4) return add ? nvec >= 2048 : nvec >= 1024;
    if (add) return (nvec > 128 && nvec <= 512) || nvec > 640;
    return nvec >= 256;
}

template <typename K>
int resident_ctas(K kernel, int block, std::atomic<int>* cache /* [kMaxDevices] */, int device) {
    int v = cache[device].load(std::memory_order_relaxed);
    if (v > 0) return v;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, block, 0) != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        n = 1;
    }
    cache[device].store(n, std::memory_order_relaxed);   // idempotent: racing first calls store the same value
    return n;
}

template <typename T, int I, bool ADD = false>
struct RegKernels {
    static constexpr int TPR = kRegShapes[I].tpr;
    static constexpr int VPT = kRegShapes[I].vpt;
    static constexpr int BLOCK = RegGeom<TPR>::kBlock;
    static constexpr int G = RegGeom<TPR>::kGroups;
    static constexpr int BWD_BLOCK = BwdGeom<TPR, VPT>::kBlock;
    static constexpr int BWD_G = BwdGeom<TPR, VPT>::kGroups;
    static constexpr bool WSM = kRegShapes[I].fat_wsm || (ADD && kRegShapes[I].wsm_add);
    // Forward with the weights in shared memory: always for the residual-add form of the shapes marked wsm_add; for
    // the plain forward of the shapes marked fwd_wsm when the type is 16-bit and every CTA makes two passes or more
    // (measured, bf16 / fp16 hidden 4096: 0.98 against 0.96 at 131 072 rows, 13.6 against 14.0 us at 4096 rows, but
    // 3.4 against 3.1 us at 256 rows, where the fill and its barrier are not hidden; fp32 hidden 2048 loses 1-5 %).
    static constexpr bool FWD_WSM_ALWAYS = ADD && kRegShapes[I].wsm_add && kRegShapes[I].fwd_ok;
    static constexpr bool FWD_WSM_LARGE = !FWD_WSM_ALWAYS && kRegShapes[I].fwd_wsm && sizeof(T) == 2;
    static bool fwd_wsm(int64_t rows, const DeviceInfo& di) {
        if constexpr (FWD_WSM_ALWAYS) return true;
        if constexpr (FWD_WSM_LARGE) return (rows + G - 1) / G >= 8ll * di.sm_count;
        return false;
    }
    // Which backward kernel this problem runs: the table's choice unless MGR_RMSNORM_BWD_FAT pins it. A problem with
    // too few rows to give every group of every fat CTA a few of them stays with one CTA per row group (2048 x 512
    // bf16: 5.1 us against 5.4 us).
    static bool fat_bwd(int64_t rows, const DeviceInfo& di) {
        if (WSM && rows >= (1ll << 31) - (1ll << 24)) return false;   // rms_bwd_wsm counts rows in 32 bits
        const int pinned = overrides().bwd_fat;
        if (pinned >= 0) return pinned != 0;
        if (WSM) return true;
        return kRegShapes[I].fat_bwd && rows >= 4ll * BWD_G * di.sm_count;
    }

    static int64_t fwd_grid(int64_t rows, const DeviceInfo& di) {
        static std::atomic<int> occ[kMaxDevices];
        static std::atomic<int> occ_wsm[kMaxDevices];
        const int64_t ngroups = (rows + G - 1) / G;
        int resident;
        if (fwd_wsm(rows, di)) {
            if constexpr (FWD_WSM_ALWAYS || FWD_WSM_LARGE) resident = resident_ctas(rms_fwd_reg<T, TPR, VPT, ADD, true>, BLOCK, occ_wsm, di.device);
            else resident = 1;   // not reached
        } else {
            if constexpr (!FWD_WSM_ALWAYS) resident = resident_ctas(rms_fwd_reg<T, TPR, VPT, ADD, false>, BLOCK, occ, di.device);
            else resident = 1;   // not reached
        }
        const int64_t cap = static_cast<int64_t>(di.sm_count) * resident;
        return ngroups < cap ? ngroups : cap;
    }
    static int64_t bwd_grid(int64_t rows, const DeviceInfo& di) {
        static std::atomic<int> occ[kMaxDevices];
        static std::atomic<int> occ_fat[kMaxDevices];
        if (fat_bwd(rows, di)) {
            const int64_t ngroups = (rows + BWD_G - 1) / BWD_G;
            int resident;
            if constexpr (WSM) resident = resident_ctas(rms_bwd_wsm<T, TPR, VPT, ADD>, BWD_BLOCK, occ_fat, di.device);
            else resident = resident_ctas(rms_bwd_fat<T, TPR, VPT, ADD>, BWD_BLOCK, occ_fat, di.device);
            const int64_t cap = static_cast<int64_t>(di.sm_count) * resident;
            return ngroups < cap ? ngroups : cap;
        }
        const int64_t ngroups = (rows + G - 1) / G;
        const int64_t cap = static_cast<int64_t>(di.sm_count) * resident_ctas(rms_bwd_reg<T, TPR, VPT, ADD>, BLOCK, occ, di.device);
        return ngroups < cap ? ngroups : cap;
    }
    static void fwd(T* y, float* inv, const T* x, const T* w, int64_t rows, int cols, float eps,
                    const DeviceInfo& di, cudaStream_t s, const T* res, T* h_out) {
        const unsigned grid = static_cast<unsigned>(fwd_grid(rows, di));
        const int pf = use_prefetch(false, ADD, sizeof(T), cols / Elem<T>::kVec) ? 1 : 0;
        if (fwd_wsm(rows, di)) {
            if constexpr (FWD_WSM_ALWAYS || FWD_WSM_LARGE) rms_fwd_reg<T, TPR, VPT, ADD, true><<<grid, BLOCK, 0, s>>>(y, inv, x, w, rows, cols, eps, res, h_out, pf);
        } else {
            if constexpr (!FWD_WSM_ALWAYS) rms_fwd_reg<T, TPR, VPT, ADD, false><<<grid, BLOCK, 0, s>>>(y, inv, x, w, rows, cols, eps, res, h_out, pf);
        }
    }
    static void bwd(T* dx, float* ws, const T* dy, const T* x, const T* w, const float* inv, int64_t rows,
                    int cols, int64_t grid, const DeviceInfo& di, cudaStream_t s, const T* dres) {
        const int pf = use_prefetch(true, ADD, sizeof(T), cols / Elem<T>::kVec) ? 1 : 0;
        if (fat_bwd(rows, di)) {
            if constexpr (WSM)
                rms_bwd_wsm<T, TPR, VPT, ADD><<<static_cast<unsigned>(grid), BWD_BLOCK, 0, s>>>(dx, ws, dy, x, w, inv, static_cast<int>(rows), cols, dres, pf);
            else
                rms_bwd_fat<T, TPR, VPT, ADD><<<static_cast<unsigned>(grid), BWD_BLOCK, 0, s>>>(dx, ws, dy, x, w, inv, rows, cols, dres, pf);
        } else
            rms_bwd_reg<T, TPR, VPT, ADD><<<static_cast<unsigned>(grid), BLOCK, 0, s>>>(dx, ws, dy, x, w, inv, rows, cols, dres, pf);
    }
};

// `res`/`h_out` (forward) and `dres` (backward) select the residual-add kernels when non-null.
template <typename T, int I = 0>
struct RegDispatch {
    static void fwd(int shape, T* y, float* inv, const T* x, const T* w, int64_t rows, int cols, float eps,
                    const DeviceInfo& di, cudaStream_t s, const T* res = nullptr, T* h_out = nullptr) {
        if (shape == I) {
            if (res != nullptr) RegKernels<T, I, true>::fwd(y, inv, x, w, rows, cols, eps, di, s, res, h_out);
            else RegKernels<T, I, false>::fwd(y, inv, x, w, rows, cols, eps, di, s, nullptr, nullptr);
        } else if constexpr (I + 1 < kNumRegShapes) {
            RegDispatch<T, I + 1>::fwd(shape, y, inv, x, w, rows, cols, eps, di, s, res, h_out);
        }
    }
    static int64_t bwd_grid(int shape, int64_t rows, const DeviceInfo& di, bool add = false) {
        if (shape == I) return add ? RegKernels<T, I, true>::bwd_grid(rows, di) : RegKernels<T, I, false>::bwd_grid(rows, di);
        if constexpr (I + 1 < kNumRegShapes) return RegDispatch<T, I + 1>::bwd_grid(shape, rows, di, add);
        return 0;
    }
    static void bwd(int shape, T* dx, float* ws, const T* dy, const T* x, const T* w, const float* inv,
                    int64_t rows, int cols, int64_t grid, const DeviceInfo& di, cudaStream_t s, const T* dres = nullptr) {
        if (shape == I) {
            if (dres != nullptr) RegKernels<T, I, true>::bwd(dx, ws, dy, x, w, inv, rows, cols, grid, di, s, dres);
            else RegKernels<T, I, false>::bwd(dx, ws, dy, x, w, inv, rows, cols, grid, di, s, nullptr);
        } else if constexpr (I + 1 < kNumRegShapes) {
            RegDispatch<T, I + 1>::bwd(shape, dx, ws, dy, x, w, inv, rows, cols, grid, di, s, dres);
        }
    }
};

int64_t scalar_grid(int64_t rows, const DeviceInfo& di) {
    const int64_t cap = static_cast<int64_t>(di.sm_count) * 8;
    return rows < cap ? rows : cap;
}

// ---- ring (bulk-copy) path ------------------------------------------------------------------------

enum class Path { kAuto, kReg, kRing, kScalar };

// MGR_RMSNORM_PATH=reg|ring|scalar pins the kernel family (benchmarking and tests); unset = automatic.
Path forced_path() {
    switch (overrides().rms_path) {
        case 1: return Path::kReg;
        case 2: return Path::kRing;
        case 3: return Path::kScalar;
        default: return Path::kAuto;
    }
}

int* rms_status_ptr(const DeviceInfo& di) {
    static std::atomic<int*> cache[kMaxDevices];
    if (cache[di.device].load(std::memory_order_relaxed) == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_rms_status) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        cache[di.device].store(static_cast<int*>(p), std::memory_order_relaxed);
    }
    return cache[di.device].load(std::memory_order_relaxed);
}

template <typename K>
bool allow_big_smem(K kernel, std::atomic<bool>* done /* [kMaxDevices] */, int device) {
    if (done[device].load(std::memory_order_acquire)) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBudget)) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    done[device].store(true, std::memory_order_release);
    return true;
}

// Returns MGR_OK if launched, 1 if the ring path does not apply (caller falls back), < 0 on error.
template <typename T>
int fwd_ring_try(T* y, float* inv, const T* x, const T* w, int64_t rows, int64_t cols, float eps, const DeviceInfo& di,
                 cudaStream_t s) {
    static std::atomic<bool> attr[kMaxDevices];
    const RingPlan plan = fwd_ring_plan(rows, cols, sizeof(T));
    if (!plan.ok) return 1;
    int* status = rms_status_ptr(di);
    if (status == nullptr || !allow_big_smem(rms_fwd_ring<T, kFwdRingWarps>, attr, di.device)) return 1;
    const int64_t nchunks = (rows + plan.rows_per_slot - 1) / plan.rows_per_slot;
    const unsigned grid = static_cast<unsigned>(nchunks < di.sm_count ? nchunks : di.sm_count);
    rms_fwd_ring<T, kFwdRingWarps><<<grid, (kFwdRingWarps + 1) * 32, plan.smem_bytes, s>>>(
        y, inv, x, w, rows, static_cast<int>(cols), eps, plan.rows_per_slot, plan.nslots, plan.w_bytes, plan.slot_bytes, status);
    return launch_status();
}

struct RingShape {
    int tpr, vpt;
};
constexpr RingShape kRingShapes[] = {{32, 1}, {32, 2}, {64, 2}, {128, 2}, {256, 2}, {512, 2}, {512, 4}};
constexpr int kNumRingShapes = sizeof(kRingShapes) / sizeof(kRingShapes[0]);

int ring_shape_for(int64_t nvec) {
    for (int i = 0; i < kNumRingShapes; ++i)
        if (nvec <= static_cast<int64_t>(kRingShapes[i].tpr) * kRingShapes[i].vpt) return i;
    return -1;
}

struct BwdRingPlan {
    int ok, shape, nslots;
    uint32_t slot_bytes, smem_bytes;
    int64_t grid;
};

BwdRingPlan bwd_ring_plan(int64_t rows, int64_t cols, size_t elem, const DeviceInfo& di) {
    BwdRingPlan p{};
    const int64_t vec = 16 / static_cast<int64_t>(elem);
    if (cols % vec != 0) return p;
    p.shape = ring_shape_for(cols / vec);
    if (p.shape < 0) return p;
    const int G = kBwdRingThreads / kRingShapes[p.shape].tpr;
    const uint64_t slot = 2ull * G * cols * elem;
    const uint32_t fixed = 2 * 8 * kRingMaxSlots + 256;
    if (fixed + 3 * slot > kSmemBudget) return p;
    int n = static_cast<int>((kSmemBudget - fixed) / slot);
    if (n > kRingMaxSlots) n = kRingMaxSlots;
    const uint64_t fold = static_cast<uint64_t>(G - 1) * kRingShapes[p.shape].tpr * kRingShapes[p.shape].vpt * 16 * 4 / elem;
    if (fold > n * slot) return p;
    p.nslots = n;
    p.slot_bytes = static_cast<uint32_t>(slot);
    p.smem_bytes = static_cast<uint32_t>(n * slot + 2 * 8 * n);
    const int64_t ngroups = (rows + G - 1) / G;
    p.grid = ngroups < di.sm_count ? ngroups : di.sm_count;
    p.ok = 1;
    return p;
}

template <typename T, int I = 0>
struct RingDispatch {
    static int bwd(const BwdRingPlan& plan, T* dx, float* ws, const T* dy, const T* x, const T* w, const float* inv,
                   int64_t rows, int cols, int* status, const DeviceInfo& di, cudaStream_t s) {
        if (plan.shape == I) {
            constexpr int TPR = kRingShapes[I].tpr, VPT = kRingShapes[I].vpt;
            static std::atomic<bool> attr[kMaxDevices];
            if (!allow_big_smem(rms_bwd_ring<T, TPR, VPT>, attr, di.device)) return 1;
            rms_bwd_ring<T, TPR, VPT><<<static_cast<unsigned>(plan.grid), kBwdRingThreads, plan.smem_bytes, s>>>(
                dx, ws, dy, x, w, inv, rows, cols, plan.nslots, plan.slot_bytes, status);
            return launch_status();
        }
        if constexpr (I + 1 < kNumRingShapes)
            return RingDispatch<T, I + 1>::bwd(plan, dx, ws, dy, x, w, inv, rows, cols, status, di, s);
        return 1;
    }
};

// Automatic choice between the register and the ring family, from back-to-back timings on B200
// (fraction of the measured 6.55 TB/s copy bandwidth, register / ring):
//   forward : 4 KB rows 0.85 / 1.00 (2 KB rows: see prefer_ring_fwd); 8 KB 0.97 / 0.95; 16 KB 0.99 / 0.92; 32 KB 0.97 / 0.89
//   backward: 2 KB rows 0.90 / 0.80; 4 KB 0.93 / 0.84; 8 KB 0.92 / 0.83; 16 KB 0.92 / 0.82; 32 KB 0.84-0.87 / 0.90-0.94
//   (register figures with the per-size packet shapes of bwd_shape_for)
// The ring needs enough rows to fill its pipeline, hence the row-count floor.
bool prefer_ring_fwd(int64_t rows, int64_t cols, size_t elem, const DeviceInfo& di) {
    const int64_t row_bytes = cols * static_cast<int64_t>(elem);
    // 2 KB rows: fp32 0.92 register / 0.97 ring; bf16 and fp16 0.95 register / 0.87 ring
    const bool from = row_bytes > 2048 || (row_bytes == 2048 && elem == 4);
    // The ring pays about 4 us to come up (a 200 KB ring per SM to fill before the first row is normalised), which a
    // small tensor never earns back. Measured (register / ring, forward, us): bf16 2048 x 2048 5.4 / 8.5; 4096 x 2048
    // 8.3 / 10.5; 16 384 x 2048 26.1 / 26.7; 65 536 x 2048 94.0 / 88.4; fp32 4096 x 512 4.6 / 8.6; 65 536 x 512
    // 46.9 / 47.7. fp32 rows of 4 KB stay with the register kernels at every size measured (131 072 x 1024: 0.93
    // against 0.90 of the copy bandwidth).
    const int64_t min_bytes = elem == 4 ? (256ll << 20) : (128ll << 20);
    if (elem == 4 && row_bytes > 2048) return false;
    return rows >= 8ll * di.sm_count && rows * row_bytes >= min_bytes && from && row_bytes <= 4096;
}
bool prefer_ring_bwd(int64_t rows, int64_t cols, size_t elem, const DeviceInfo& di) {
    const int64_t row_bytes = cols * static_cast<int64_t>(elem);
    // Rows of 16-24 KB (1025-1536 packets) have a packet shape of their own, {384,4}: bf16 hidden 12 288 at 16 384 rows
    // 0.75 with it against 0.69 for the ring (2048 rows: 0.59 against 0.55). Beyond that the ring is ahead at every
    // row count measured (32 KB rows, 2048 to 32 768 rows: 0.66-0.90 against 0.65-0.84; fp32 0.86-0.98 against 0.74-0.87).
    // With the next row requested into L2 ahead of time the {512,4} packet kernel passes the ring at 32 KB rows of a
    // 16-bit type as well (bf16 hidden 16 384: 0.95 against 0.87; 2048 rows: 0.74 against 0.66); fp32 rows of 32 KB
    // stay with the ring (1.07 against 1.05), and so do rows beyond 32 KB (equal at 64 KB: 0.95 / 0.94).
    return rows >= 8ll * di.sm_count && row_bytes > (elem == 4 ? 24576 : 32768);
}

template <typename T>
int fwd_typed(void* y, float* inv, const void* x, const void* w, int64_t rows, int64_t cols, float eps,
              const DeviceInfo& di, cudaStream_t s, const void* res = nullptr, void* h_out = nullptr) {
    constexpr int VEC = Elem<T>::kVec;
    const Path forced = forced_path();
    const bool add = res != nullptr;   // the residual-add variants exist in the register and scalar families
    const bool packets = forced != Path::kScalar && cols % VEC == 0 && aligned_to(y, 16) && aligned_to(x, 16) && aligned_to(w, 16) &&
                         aligned_to(res, 16) && aligned_to(h_out, 16);
    if (!add && y != nullptr && packets && forced != Path::kReg && (forced == Path::kRing || prefer_ring_fwd(rows, cols, sizeof(T), di))) {
        const int st = fwd_ring_try<T>(static_cast<T*>(y), inv, static_cast<const T*>(x), static_cast<const T*>(w), rows, cols, eps, di, s);
        if (st <= 0) return st;
    }
    const int shape = packets ? fwd_shape_for(cols / VEC) : -1;
    if (shape >= 0) {
        RegDispatch<T>::fwd(shape, static_cast<T*>(y), inv, static_cast<const T*>(x), static_cast<const T*>(w), rows,
                            static_cast<int>(cols), eps, di, s, static_cast<const T*>(res), static_cast<T*>(h_out));
    } else if (add) {
        rms_fwd_scalar<T, true><<<static_cast<unsigned>(scalar_grid(rows, di)), 256, 0, s>>>(
            static_cast<T*>(y), inv, static_cast<const T*>(x), static_cast<const T*>(w), rows, cols, eps,
            static_cast<const T*>(res), static_cast<T*>(h_out));
    } else {
        rms_fwd_scalar<T><<<static_cast<unsigned>(scalar_grid(rows, di)), 256, 0, s>>>(
            static_cast<T*>(y), inv, static_cast<const T*>(x), static_cast<const T*>(w), rows, cols, eps);
    }
    return launch_status();
}

// Partial rows the backward of this problem may write: the largest over the three kernel families,
// so one workspace size serves whichever family the pointers and the policy select.
template <typename T>
int64_t bwd_partials(int64_t rows, int64_t cols, const DeviceInfo& di) {
    constexpr int VEC = Elem<T>::kVec;
    int64_t p = rows < kScalarDwSlices ? rows : kScalarDwSlices;
    if (cols % VEC == 0) {
        const int shape = bwd_shape_for(cols / VEC);
        if (shape >= 0) {
            const int64_t g = RegDispatch<T>::bwd_grid(shape, rows, di);
            if (g > p) p = g;
        }
        const int shape_add = bwd_shape_for(cols / VEC, sizeof(T) == 2);
        if (shape_add >= 0) {
            const int64_t ga = RegDispatch<T>::bwd_grid(shape_add, rows, di, true);
            if (ga > p) p = ga;
        }
        const BwdRingPlan rp = bwd_ring_plan(rows, cols, sizeof(T), di);
        if (rp.ok && rp.grid > p) p = rp.grid;
    }
    return p < 1 ? 1 : p;
}

template <typename T>
int bwd_typed(void* dx, void* dw, float* dw_f32, const void* dy, const void* x, const void* w, const float* inv,
              int64_t rows, int64_t cols, float* ws, const DeviceInfo& di, cudaStream_t s, const void* dres = nullptr) {
    constexpr int VEC = Elem<T>::kVec;
    const Path forced = forced_path();
    const bool add = dres != nullptr;
    const bool packets = forced != Path::kScalar && cols % VEC == 0 && aligned_to(dx, 16) && aligned_to(dy, 16) &&
                         aligned_to(x, 16) && aligned_to(w, 16) && aligned_to(dres, 16);
    int64_t P = -1;
    if (!add && packets && forced != Path::kReg && (forced == Path::kRing || prefer_ring_bwd(rows, cols, sizeof(T), di))) {
        const BwdRingPlan plan = bwd_ring_plan(rows, cols, sizeof(T), di);
        int* status = plan.ok ? rms_status_ptr(di) : nullptr;
        if (status != nullptr) {
            const int st = RingDispatch<T>::bwd(plan, static_cast<T*>(dx), ws, static_cast<const T*>(dy), static_cast<const T*>(x),
                                                static_cast<const T*>(w), inv, rows, static_cast<int>(cols), status, di, s);
            if (st < 0) return st;
            if (st == 0) P = plan.grid;
        }
    }
    if (P < 0) {
        const int shape = packets ? bwd_shape_for(cols / VEC, add && sizeof(T) == 2) : -1;
        if (shape >= 0) {
            P = RegDispatch<T>::bwd_grid(shape, rows, di, add);
            RegDispatch<T>::bwd(shape, static_cast<T*>(dx), ws, static_cast<const T*>(dy), static_cast<const T*>(x),
                                static_cast<const T*>(w), inv, rows, static_cast<int>(cols), P, di, s, static_cast<const T*>(dres));
        } else {
            P = rows < kScalarDwSlices ? rows : kScalarDwSlices;
            if (add)
                rms_bwd_dx_scalar<T, true><<<static_cast<unsigned>(scalar_grid(rows, di)), 256, 0, s>>>(
                    static_cast<T*>(dx), static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(w), inv, rows, cols,
                    static_cast<const T*>(dres));
            else
                rms_bwd_dx_scalar<T><<<static_cast<unsigned>(scalar_grid(rows, di)), 256, 0, s>>>(
                    static_cast<T*>(dx), static_cast<const T*>(dy), static_cast<const T*>(x), static_cast<const T*>(w), inv, rows, cols);
            int st = launch_status();
            if (st != MGR_OK) return st;
            dim3 grid(static_cast<unsigned>((cols + 127) / 128), static_cast<unsigned>(P));
            rms_bwd_dw_scalar<T><<<grid, 128, 0, s>>>(ws, static_cast<const T*>(dy), static_cast<const T*>(x), inv, rows, cols);
        }
        int st = launch_status();
        if (st != MGR_OK) return st;
    }
    // Programmatic dependent launch: the reduce is queued behind the backward kernel without waiting for the
    // stream to go idle in between, which hides its launch latency (a few microseconds; it matters for the
    // 10-30 us problems).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>((cols + 31) / 32));
    cfg.blockDim = dim3(32, 32);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    if (cols % 4 == 0) {   // rows of the workspace start on 16-byte boundaries: the packet form of the column sum
        cfg.blockDim = dim3(1024);
        if (cudaLaunchKernelEx(&cfg, rms_dw_reduce4<T>, static_cast<T*>(dw), dw_f32, static_cast<const float*>(ws), static_cast<int>(P),
                               static_cast<int>(cols)) == cudaSuccess)
            return launch_status();
        (void)cudaGetLastError();
        cfg.blockDim = dim3(32, 32);
    }
    if (cudaLaunchKernelEx(&cfg, rms_dw_reduce<T>, static_cast<T*>(dw), dw_f32, static_cast<const float*>(ws), static_cast<int>(P),
                           static_cast<int>(cols)) != cudaSuccess) {
        (void)cudaGetLastError();
        rms_dw_reduce<T><<<static_cast<unsigned>((cols + 31) / 32), dim3(32, 32), 0, s>>>(
            static_cast<T*>(dw), dw_f32, ws, static_cast<int>(P), static_cast<int>(cols));
    }
    return launch_status();
}

int check_common(int64_t rows, int64_t cols, int dtype) {
    if (dtype_size(dtype) == 0) return MGR_ERR_BAD_DTYPE;
    if (rows < 0 || cols < 1) return MGR_ERR_BAD_SHAPE;
    if (cols > (1ll << 30) || rows > (1ll << 40)) return MGR_ERR_TOO_LARGE;
    return MGR_OK;
}

}  // namespace
}  // namespace mgr

using namespace mgr;

namespace mgr {
namespace {
// Shared by the plain and the residual-add forward; `add` says which (then res and h_out are required).
int fwd_entry(void* y, float* inv_rms, const void* x, const void* w, int64_t rows, int64_t cols, float eps, int dtype,
              void* stream, bool add, const void* res, void* h_out, bool inv_only = false) {
    int st = check_common(rows, cols, dtype);
    if (st != MGR_OK) return st;
    if (rows == 0) return MGR_OK;
    if (inv_only) {            // no output tensor and no weight: the kernels skip the stores, and read x as the "weight"
        if (inv_rms == nullptr) return MGR_ERR_NULL_PTR;
        y = nullptr;
        w = x;
    } else if (y == nullptr) {
        return MGR_ERR_NULL_PTR;
    }
    if (x == nullptr || w == nullptr) return MGR_ERR_NULL_PTR;
    if (add && (res == nullptr || h_out == nullptr)) return MGR_ERR_NULL_PTR;
    const size_t es = dtype_size(dtype);
    if (!aligned_to(y, es) || !aligned_to(x, es) || !aligned_to(w, es) || !aligned_to(inv_rms, 4)) return MGR_ERR_MISALIGNED;
    if (add && (!aligned_to(res, es) || !aligned_to(h_out, es))) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (!add) res = nullptr, h_out = nullptr;
    switch (dtype) {
        case MGR_F32: return fwd_typed<float>(y, inv_rms, x, w, rows, cols, eps, di, s, res, h_out);
        case MGR_F16: return fwd_typed<__half>(y, inv_rms, x, w, rows, cols, eps, di, s, res, h_out);
        default: return fwd_typed<__nv_bfloat16>(y, inv_rms, x, w, rows, cols, eps, di, s, res, h_out);
    }
}
}  // namespace
}  // namespace mgr

extern "C" int mgr_rmsnorm_fwd(void* y, float* inv_rms, const void* x, const void* w, int64_t rows, int64_t cols,
                               float eps, int dtype, void* stream) {
    return fwd_entry(y, inv_rms, x, w, rows, cols, eps, dtype, stream, false, nullptr, nullptr);
}

extern "C" int mgr_rms_inv(float* inv_rms, const void* x, int64_t rows, int64_t cols, float eps, int dtype, void* stream) {
    return fwd_entry(nullptr, inv_rms, x, nullptr, rows, cols, eps, dtype, stream, false, nullptr, nullptr, true);
}

extern "C" int mgr_add_rmsnorm_fwd(void* y, void* h, float* inv_rms, const void* x, const void* residual, const void* w,
                                   int64_t rows, int64_t cols, float eps, int dtype, void* stream) {
    return fwd_entry(y, inv_rms, x, w, rows, cols, eps, dtype, stream, true, residual, h);
}

extern "C" size_t mgr_rmsnorm_bwd_workspace_bytes(int64_t rows, int64_t cols, int dtype) {
    if (check_common(rows, cols, dtype) != MGR_OK) return 0;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return 0;
    int64_t p;
    switch (dtype) {
        case MGR_F32: p = bwd_partials<float>(rows, cols, di); break;
        case MGR_F16: p = bwd_partials<__half>(rows, cols, di); break;
        default: p = bwd_partials<__nv_bfloat16>(rows, cols, di); break;
    }
    return static_cast<size_t>(p) * static_cast<size_t>(cols) * sizeof(float);
}

namespace mgr {
namespace {
int bwd_entry(void* dx, void* dw, float* dw_f32, const void* dy, const void* x, const void* w, const float* inv_rms,
              int64_t rows, int64_t cols, int dtype, void* workspace, size_t workspace_bytes, void* stream, bool add,
              const void* dres) {
    int st = check_common(rows, cols, dtype);
    if (st != MGR_OK) return st;
    if (dw == nullptr && dw_f32 == nullptr) return MGR_ERR_NULL_PTR;
    const size_t es = dtype_size(dtype);
    if (!aligned_to(dw, es) || !aligned_to(dw_f32, 4)) return MGR_ERR_MISALIGNED;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (rows == 0) {
        if (dw != nullptr && cudaMemsetAsync(dw, 0, static_cast<size_t>(cols) * es, s) != cudaSuccess) return MGR_ERR_CUDA;
        if (dw_f32 != nullptr && cudaMemsetAsync(dw_f32, 0, static_cast<size_t>(cols) * 4, s) != cudaSuccess) return MGR_ERR_CUDA;
        return MGR_OK;
    }
    if (dx == nullptr || dy == nullptr || x == nullptr || w == nullptr || inv_rms == nullptr || workspace == nullptr)
        return MGR_ERR_NULL_PTR;
    if (add && dres == nullptr) return MGR_ERR_NULL_PTR;
    if (!aligned_to(dx, es) || !aligned_to(dy, es) || !aligned_to(x, es) || !aligned_to(w, es) ||
        !aligned_to(inv_rms, 4) || !aligned_to(workspace, 16) || (add && !aligned_to(dres, es)))
        return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    if (workspace_bytes < mgr_rmsnorm_bwd_workspace_bytes(rows, cols, dtype)) return MGR_ERR_WORKSPACE_TOO_SMALL;
    float* ws = static_cast<float*>(workspace);
    if (!add) dres = nullptr;
    switch (dtype) {
        case MGR_F32: return bwd_typed<float>(dx, dw, dw_f32, dy, x, w, inv_rms, rows, cols, ws, di, s, dres);
        case MGR_F16: return bwd_typed<__half>(dx, dw, dw_f32, dy, x, w, inv_rms, rows, cols, ws, di, s, dres);
        default: return bwd_typed<__nv_bfloat16>(dx, dw, dw_f32, dy, x, w, inv_rms, rows, cols, ws, di, s, dres);
    }
}
}  // namespace
}  // namespace mgr

extern "C" int mgr_rmsnorm_bwd(void* dx, void* dw, float* dw_f32, const void* dy, const void* x, const void* w,
                               const float* inv_rms, int64_t rows, int64_t cols, int dtype, void* workspace,
                               size_t workspace_bytes, void* stream) {
    return bwd_entry(dx, dw, dw_f32, dy, x, w, inv_rms, rows, cols, dtype, workspace, workspace_bytes, stream, false, nullptr);
}

extern "C" int mgr_add_rmsnorm_bwd(void* dh, void* dw, float* dw_f32, const void* dy, const void* dres, const void* h,
                                   const void* w, const float* inv_rms, int64_t rows, int64_t cols, int dtype,
                                   void* workspace, size_t workspace_bytes, void* stream) {
    return bwd_entry(dh, dw, dw_f32, dy, h, w, inv_rms, rows, cols, dtype, workspace, workspace_bytes, stream, true, dres);
}

// Defined here, declared for capi_common.cu: reads (and optionally clears) this file's status word.
namespace mgr {
int rmsnorm_status_fetch(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_rms_status, sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        return MGR_ERR_CUDA;
    }
    if (clear && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_rms_status, &zero, sizeof(int)) != cudaSuccess) (void)cudaGetLastError();
    }
    return v;
}

int rmsnorm_status_poke(int value) {
    return cudaMemcpyToSymbol(g_rms_status, &value, sizeof(int)) == cudaSuccess ? MGR_OK : ((void)cudaGetLastError(), MGR_ERR_CUDA);
}
}  // namespace mgr

// ------------------------------------------------------------------------------------------------
// Backward for callers that cannot allocate device memory.
//
// mgr_rmsnorm_bwd takes its scratch (the per-CTA fp32 partial rows of dW) from the caller. A caller
// that has no allocator to ask -- a plain C/C++ host without torch's caching allocator, or a serving
// loop that must not call cudaMalloc once it is running, because cudaMalloc and cudaFree synchronise
// the whole device and can fail late through fragmentation -- uses this entry point instead: the
// scratch is a fixed array that lives in the library's device image.
//
// The array is part of every context that loads the library (16 MiB per GPU until the process exits).
// All calls on a device share it and it keeps the previous call's partial rows; nothing in it has to
// start at zero, because the backward kernel overwrites every partial row the reduce kernel then reads.
// Two calls that overlap on the GPU (different streams, no ordering between them) race on the array.
// ------------------------------------------------------------------------------------------------

static __device__ __align__(256) float g_noalloc_scratch[MGR_NOALLOC_SCRATCH_BYTES / sizeof(float)];

namespace mgr {
namespace {

// Device address of g_noalloc_scratch on the CURRENT device. In host code the array's name is only a
// handle for the runtime, not an address a kernel can use: the address comes from
// cudaGetSymbolAddress, asked once per device with that device current, and is cached.
float* noalloc_scratch(const DeviceInfo& di) {
    static std::atomic<float*> cache[kMaxDevices];   // racing first calls store the same address
    float* known = cache[di.device].load(std::memory_order_relaxed);
    if (known == nullptr) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            (void)cudaGetLastError();
            return nullptr;
        }
        known = static_cast<float*>(p);
        cache[di.device].store(known, std::memory_order_relaxed);
    }
    return known;
}

}  // namespace
}  // namespace mgr

extern "C" int mgr_rmsnorm_bwd_noalloc(void* dx, void* dw, float* dw_f32, const void* dy, const void* x, const void* w,
                                       const float* inv_rms, int64_t rows, int64_t cols, int dtype, void* stream) {
    const int st = check_common(rows, cols, dtype);
    if (st != MGR_OK) return st;
    if (rows == 0)  // nothing to reduce: the scratch is not touched
        return mgr_rmsnorm_bwd(dx, dw, dw_f32, dy, x, w, inv_rms, rows, cols, dtype, nullptr, 0, stream);
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    const size_t need = mgr_rmsnorm_bwd_workspace_bytes(rows, cols, dtype);
    if (need == 0) return MGR_ERR_CUDA;
    if (need > MGR_NOALLOC_SCRATCH_BYTES) return MGR_ERR_TOO_LARGE;
    float* scratch = noalloc_scratch(di);
    if (scratch == nullptr) return MGR_ERR_CUDA;
    return mgr_rmsnorm_bwd(dx, dw, dw_f32, dy, x, w, inv_rms, rows, cols, dtype, scratch, MGR_NOALLOC_SCRATCH_BYTES, stream);
}
