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

__device__ __forceinline__ float sigmoidf_(float g) { return 1.0f / (1.0f + __expf(-g)); }

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_act_fwd_packets(T* __restrict__ h, const T* __restrict__ gv, int64_t m, int64_t fpk /* packets per row of h */) {
    constexpr int VEC = Elem<T>::kVec;
    const int64_t total = m * fpk;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const uint4* in = reinterpret_cast<const uint4*>(gv);
    uint4* out = reinterpret_cast<uint4*>(h);
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / fpk;
        const int64_t c = idx - row * fpk;
        const uint4 pg = ld_stream16(in + row * 2 * fpk + c);
        const uint4 pv = ld_stream16(in + row * 2 * fpk + fpk + c);
        float g[VEC], v[VEC], o[VEC];
        unpack16<T>(pg, g);
        unpack16<T>(pv, v);
#pragma unroll
        for (int i = 0; i < VEC; ++i) o[i] = (g[i] * sigmoidf_(g[i])) * v[i];
        st_stream16(out + idx, pack16<T>(o));
    }
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_act_bwd_packets(T* __restrict__ dgv, const T* __restrict__ dh, const T* __restrict__ gv, int64_t m, int64_t fpk) {
    constexpr int VEC = Elem<T>::kVec;
    const int64_t total = m * fpk;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const uint4* in = reinterpret_cast<const uint4*>(gv);
    const uint4* gin = reinterpret_cast<const uint4*>(dh);
    uint4* out = reinterpret_cast<uint4*>(dgv);
    for (int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int64_t row = idx / fpk;
        const int64_t c = idx - row * fpk;
        const uint4 pg = ld_stream16(in + row * 2 * fpk + c);
        const uint4 pv = ld_stream16(in + row * 2 * fpk + fpk + c);
        const uint4 po = ld_stream16(gin + idx);
        float g[VEC], v[VEC], go[VEC], dg[VEC], dv[VEC];
        unpack16<T>(pg, g);
        unpack16<T>(pv, v);
        unpack16<T>(po, go);
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float sig = sigmoidf_(g[i]);
            dv[i] = go[i] * (g[i] * sig);
            dg[i] = go[i] * v[i] * (sig * (1.0f + g[i] * (1.0f - sig)));
        }
        st_stream16(out + row * 2 * fpk + c, pack16<T>(dg));
        st_stream16(out + row * 2 * fpk + fpk + c, pack16<T>(dv));
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
        h[idx] = from_f32<T>((g * sigmoidf_(g)) * v);
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
        const float sig = sigmoidf_(g);
        dgv[row * 2 * f + c] = from_f32<T>(go * v * (sig * (1.0f + g * (1.0f - sig))));
        dgv[row * 2 * f + f + c] = from_f32<T>(go * (g * sig));
    }
}

unsigned flat_grid(int64_t work_items, const DeviceInfo& di) {
    const int64_t need = (work_items + 255) / 256;
    const int64_t cap = static_cast<int64_t>(di.sm_count) * 8;  // 8 x 256 threads = a full SM
    const int64_t g = need < cap ? need : cap;
    return static_cast<unsigned>(g < 1 ? 1 : g);
}

template <typename T>
int act_fwd_typed(void* h, const void* gv, int64_t m, int64_t f, const DeviceInfo& di, cudaStream_t s) {
    constexpr int VEC = Elem<T>::kVec;
    if (f % VEC == 0 && aligned_to(h, 16) && aligned_to(gv, 16)) {
        const int64_t fpk = f / VEC;
        swiglu_act_fwd_packets<T><<<flat_grid(m * fpk, di), 256, 0, s>>>(static_cast<T*>(h), static_cast<const T*>(gv), m, fpk);
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
        swiglu_act_bwd_packets<T><<<flat_grid(m * fpk, di), 256, 0, s>>>(static_cast<T*>(dgv), static_cast<const T*>(dh),
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
