// Stand-alone SwiGLU activation, forward and backward, for sm_100a.
//
// Replaces the reference's two Triton kernels, _mg_swiglu_fwd_kernel and _mg_swiglu_bwd_kernel
// (megagemm/swiglu.py:18-43, 46-79), which MegaGemmFunction launches one program per row. Same
// arithmetic: fp32 math on values loaded in the tensor dtype, one rounding on store. Both are pure
// HBM streams, so the kernels here are flat grid-stride loops over 16-byte packets sized to the SM
// count. (The MLP's fast path does not run them: there the product is fused into the GEMM epilogue.)

#include "mgr_common.cuh"

namespace mgr {
namespace {

// 16-bit types: MUFU exp + MUFU reciprocal (about 2 ulp in fp32, far below the rounding of the output). With an IEEE
// division the 16-bit kernels, which do twice the arithmetic per byte of the fp32 ones, were held back by it: fp16
// and bf16 forward 0.87 of the copy bandwidth with the division, 0.97 without (65 536 x 6912; 4096 rows: 0.78 -> 0.90).
// fp32 keeps the division: it runs at 0.99 with it and measured 0.95 without.
template <typename T>
__device__ __forceinline__ float sigmoidf_(float g) {
    if constexpr (sizeof(T) == 2) return __fdividef(1.0f, 1.0f + __expf(-g));
    else return 1.0f / (1.0f + __expf(-g));
}

// Position of a flat packet index inside the [m, fpk] grid of h, advanced by a fixed stride without dividing:
// the stride is split once into whole rows and a remainder.
struct PacketPos {
    int64_t row, c;
    __device__ __forceinline__ void advance(int64_t q, int64_t r, int64_t fpk) {
        row += q;
        c += r;
        if (c >= fpk) {
            c -= fpk;
            ++row;
        }
    }
};

template <typename T>
__device__ __forceinline__ uint4 act_fwd_packet(const uint4& pg, const uint4& pv) {
    constexpr int VEC = Elem<T>::kVec;
    float g[VEC], v[VEC], o[VEC];
    unpack16<T>(pg, g);
    unpack16<T>(pv, v);
#pragma unroll
    for (int i = 0; i < VEC; ++i) o[i] = (g[i] * sigmoidf_<T>(g[i])) * v[i];
    return pack16<T>(o);
}

// Two grid-stride positions per turn: the four loads of both are issued before either is used (a thread with
// two 16-byte loads in flight kept the stream at 0.65 of the copy bandwidth, with four it reaches the backward's 0.86+).
template <typename T>
__global__ void __launch_bounds__(256, 4)
swiglu_act_fwd_packets(T* __restrict__ h, const T* __restrict__ gv, int64_t m, int64_t fpk /* packets per row of h */) {
    const int64_t total = m * fpk;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t sq = stride / fpk, sr = stride - sq * fpk;
    const uint4* in = reinterpret_cast<const uint4*>(gv);
    uint4* out = reinterpret_cast<uint4*>(h);
    int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    PacketPos p{idx / fpk, idx % fpk};
    for (; idx + stride < total; idx += 2 * stride) {
        PacketPos p2 = p;
        p2.advance(sq, sr, fpk);
        const uint4 g0 = ld_stream16(in + p.row * 2 * fpk + p.c);
        const uint4 v0 = ld_stream16(in + p.row * 2 * fpk + fpk + p.c);
        const uint4 g1 = ld_stream16(in + p2.row * 2 * fpk + p2.c);
        const uint4 v1 = ld_stream16(in + p2.row * 2 * fpk + fpk + p2.c);
        st_stream16(out + idx, act_fwd_packet<T>(g0, v0));
        st_stream16(out + idx + stride, act_fwd_packet<T>(g1, v1));
        p = p2;
        p.advance(sq, sr, fpk);
    }
    if (idx < total) {
        const uint4 g0 = ld_stream16(in + p.row * 2 * fpk + p.c);
        const uint4 v0 = ld_stream16(in + p.row * 2 * fpk + fpk + p.c);
        st_stream16(out + idx, act_fwd_packet<T>(g0, v0));
    }
}

template <typename T>
__device__ __forceinline__ void act_bwd_packet(const uint4& pg, const uint4& pv, const uint4& po, uint4& dgp, uint4& dvp) {
    constexpr int VEC = Elem<T>::kVec;
    float g[VEC], v[VEC], go[VEC], dg[VEC], dv[VEC];
    unpack16<T>(pg, g);
    unpack16<T>(pv, v);
    unpack16<T>(po, go);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const float sig = sigmoidf_<T>(g[i]);
        dv[i] = go[i] * (g[i] * sig);
        dg[i] = go[i] * v[i] * (sig * (1.0f + g[i] * (1.0f - sig)));
    }
    dgp = pack16<T>(dg);
    dvp = pack16<T>(dv);
}

template <typename T>
__global__ void __launch_bounds__(256, 3)
swiglu_act_bwd_packets(T* __restrict__ dgv, const T* __restrict__ dh, const T* __restrict__ gv, int64_t m, int64_t fpk) {
    const int64_t total = m * fpk;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t sq = stride / fpk, sr = stride - sq * fpk;
    const uint4* in = reinterpret_cast<const uint4*>(gv);
    const uint4* gin = reinterpret_cast<const uint4*>(dh);
    uint4* out = reinterpret_cast<uint4*>(dgv);
    int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    PacketPos p{idx / fpk, idx % fpk};
    for (; idx + stride < total; idx += 2 * stride) {
        PacketPos p2 = p;
        p2.advance(sq, sr, fpk);
        const uint4 g0 = ld_stream16(in + p.row * 2 * fpk + p.c);
        const uint4 v0 = ld_stream16(in + p.row * 2 * fpk + fpk + p.c);
        const uint4 o0 = ld_stream16(gin + idx);
        const uint4 g1 = ld_stream16(in + p2.row * 2 * fpk + p2.c);
        const uint4 v1 = ld_stream16(in + p2.row * 2 * fpk + fpk + p2.c);
        const uint4 o1 = ld_stream16(gin + idx + stride);
        uint4 dg, dv;
        act_bwd_packet<T>(g0, v0, o0, dg, dv);
        st_stream16(out + p.row * 2 * fpk + p.c, dg);
        st_stream16(out + p.row * 2 * fpk + fpk + p.c, dv);
        act_bwd_packet<T>(g1, v1, o1, dg, dv);
        st_stream16(out + p2.row * 2 * fpk + p2.c, dg);
        st_stream16(out + p2.row * 2 * fpk + fpk + p2.c, dv);
        p = p2;
        p.advance(sq, sr, fpk);
    }
    if (idx < total) {
        const uint4 g0 = ld_stream16(in + p.row * 2 * fpk + p.c);
        const uint4 v0 = ld_stream16(in + p.row * 2 * fpk + fpk + p.c);
        const uint4 o0 = ld_stream16(gin + idx);
        uint4 dg, dv;
        act_bwd_packet<T>(g0, v0, o0, dg, dv);
        st_stream16(out + p.row * 2 * fpk + p.c, dg);
        st_stream16(out + p.row * 2 * fpk + fpk + p.c, dv);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_act_fwd_scalar(T* __restrict__ h, const T* __restrict__ gv, int64_t m, int64_t f) {
    const int64_t total = m * f;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / f, c = idx - row * f;
        const float g = to_f32(gv[row * 2 * f + c]), v = to_f32(gv[row * 2 * f + f + c]);
        h[idx] = from_f32<T>((g * sigmoidf_<T>(g)) * v);
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_act_bwd_scalar(T* __restrict__ dgv, const T* __restrict__ dh, const T* __restrict__ gv, int64_t m, int64_t f) {
    const int64_t total = m * f;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / f, c = idx - row * f;
        const float g = to_f32(gv[row * 2 * f + c]), v = to_f32(gv[row * 2 * f + f + c]), go = to_f32(dh[idx]);
        const float sig = sigmoidf_<T>(g);
        dgv[row * 2 * f + c] = from_f32<T>(go * v * (sig * (1.0f + g * (1.0f - sig))));
        dgv[row * 2 * f + f + c] = from_f32<T>(go * (g * sig));
    }
}

unsigned flat_grid(int64_t work_items, const DeviceInfo& di, int ctas_per_sm = 8) {
    const int64_t need = (work_items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(di.sm_count) * ctas_per_sm;  // 8 x 256 threads = a full SM
    const int64_t g = need < cap ? need : cap;
    return static_cast<unsigned>(g < 1 ? 1 : g);
}

template <typename T>
int act_fwd_typed(void* h, const void* gv, int64_t m, int64_t f, const DeviceInfo& di, cudaStream_t s) {
    constexpr int VEC = Elem<T>::kVec;
    if (f % VEC == 0 && aligned_to(h, 16) && aligned_to(gv, 16)) {
        const int64_t fpk = f / VEC;
        swiglu_act_fwd_packets<T><<<flat_grid(m * fpk, di, 4), 256, 0, s>>>(static_cast<T*>(h), static_cast<const T*>(gv), m, fpk);
    } else {
        swiglu_act_fwd_scalar<T><<<flat_grid(m * f, di), 256, 0, s>>>(static_cast<T*>(h), static_cast<const T*>(gv), m, f);
    }
    return launch_status();
}

template <typename T>
int act_bwd_typed(void* dgv, const void* dh, const void* gv, int64_t m, int64_t f, const DeviceInfo& di, cudaStream_t s) {
    constexpr int VEC = Elem<T>::kVec;
    if (f % VEC == 0 && aligned_to(dgv, 16) && aligned_to(dh, 16) && aligned_to(gv, 16)) {
        const int64_t fpk = f / VEC;
        swiglu_act_bwd_packets<T><<<flat_grid(m * fpk, di, 3), 256, 0, s>>>(static_cast<T*>(dgv), static_cast<const T*>(dh),
                                                                        static_cast<const T*>(gv), m, fpk);
    } else {
        swiglu_act_bwd_scalar<T><<<flat_grid(m * f, di), 256, 0, s>>>(static_cast<T*>(dgv), static_cast<const T*>(dh),
                                                                     static_cast<const T*>(gv), m, f);
    }
    return launch_status();
}

int act_check(int64_t m, int64_t f, int dtype) {
    if (dtype_size(dtype) == 0) return MGR_ERR_BAD_DTYPE;
    if (m < 0 || f < 1) return MGR_ERR_BAD_SHAPE;
    if (f > (1ll << 30) || m > (1ll << 40)) return MGR_ERR_TOO_LARGE;
    return MGR_OK;
}

}  // namespace
}  // namespace mgr

using namespace mgr;

extern "C" int mgr_swiglu_act_fwd(void* h, const void* gv, int64_t m, int64_t f, int dtype, void* stream) {
    int st = act_check(m, f, dtype);
    if (st != MGR_OK) return st;
    if (m == 0) return MGR_OK;
    if (h == nullptr || gv == nullptr) return MGR_ERR_NULL_PTR;
    const size_t es = dtype_size(dtype);
    if (!aligned_to(h, es) || !aligned_to(gv, es)) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MGR_F32: return act_fwd_typed<float>(h, gv, m, f, di, s);
        case MGR_F16: return act_fwd_typed<__half>(h, gv, m, f, di, s);
        default: return act_fwd_typed<__nv_bfloat16>(h, gv, m, f, di, s);
    }
}

extern "C" int mgr_swiglu_act_bwd(void* dgv, const void* dh, const void* gv, int64_t m, int64_t f, int dtype, void* stream) {
    int st = act_check(m, f, dtype);
    if (st != MGR_OK) return st;
    if (m == 0) return MGR_OK;
    if (dgv == nullptr || dh == nullptr || gv == nullptr) return MGR_ERR_NULL_PTR;
    const size_t es = dtype_size(dtype);
    if (!aligned_to(dgv, es) || !aligned_to(dh, es) || !aligned_to(gv, es)) return MGR_ERR_MISALIGNED;
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case MGR_F32: return act_bwd_typed<float>(dgv, dh, gv, m, f, di, s);
        case MGR_F16: return act_bwd_typed<__half>(dgv, dh, gv, m, f, di, s);
        default: return act_bwd_typed<__nv_bfloat16>(dgv, dh, gv, m, f, di, s);
    }
}
