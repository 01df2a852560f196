// Shared device/host helpers for libmgr_b200.so (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mgr_b200.h"

namespace mgr {

constexpr int kMaxDevices = 64;

// ---- host side -------------------------------------------------------------------------------

struct DeviceInfo {
    int status;    // MGR_OK, MGR_ERR_UNSUPPORTED_ARCH or MGR_ERR_CUDA
    int device;    // ordinal of the current device
    int sm_count;  // multiprocessors
};

// Properties of the CURRENT device, cached per ordinal after the first query (host only, thread-safe:
// concurrent first calls compute the same values).
DeviceInfo current_device_info();

// Measurement and test overrides read from the environment ONCE per process (first use) and again only when
// mgr_reload_env() is called, so that no launch pays for getenv:
//   MGR_RMSNORM_PATH=reg|ring|scalar   kernel family            MGR_RMSNORM_FWD_SHAPE / _BWD_SHAPE=<index>  packet shape
//   MGR_RMSNORM_BWD_FAT=0|1            backward packet kernel: one CTA per row group / one fat CTA per SM, for every shape
//   MGR_RMSNORM_PREFETCH=0|1           packet kernels: never / always ask L2 for the next row (where the kernel carries the code)
//   MGR_GEMM_CTA_GROUP=1|2             MGR_GEMM_PDL=0           MGR_GEMM_NARROW=0|1|32|96
struct Overrides {
    int rms_path;    // 0 automatic, 1 reg, 2 ring, 3 scalar
    int fwd_shape;   // -1 unset
    int bwd_shape;   // -1 unset
    int bwd_fat;     // -1 per packet shape (the table's choice), 0 never, 1 always
    int cta_group;   // 0 automatic, 1, 2
    int pdl;         // 0 off, 1 on
    int narrow;      // -1 automatic, 0 never, 64, 32, 96 (the fused projection only; others take 64)
    int prefetch;    // MGR_RMSNORM_PREFETCH: -1 automatic, 0 never, 1 always (the packet kernels' L2 request for the next row)
};
Overrides overrides();

inline size_t dtype_size(int dtype) {
    switch (dtype) {
        case MGR_F32: return 4;
        case MGR_F16: return 2;
        case MGR_BF16: return 2;
        default: return 0;
    }
}

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

// Maps the result of a kernel launch to a status code without synchronising.
inline int launch_status() {
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return MGR_OK;
    if (e == cudaErrorNoKernelImageForDevice || e == cudaErrorInvalidDeviceFunction) return MGR_ERR_UNSUPPORTED_ARCH;
    return MGR_ERR_LAUNCH_FAILED;
}

// ---- device side: 16-byte packets of T <-> fp32 ------------------------------------------------

template <typename T>
struct Elem {
    static constexpr int kVec = 16 / sizeof(T);  // elements per 16-byte packet
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T> __device__ __forceinline__ void unpack16(const uint4& p, float (&f)[Elem<T>::kVec]);

template <>
__device__ __forceinline__ void unpack16<float>(const uint4& p, float (&f)[4]) {
    f[0] = __uint_as_float(p.x);
    f[1] = __uint_as_float(p.y);
    f[2] = __uint_as_float(p.z);
    f[3] = __uint_as_float(p.w);
}

template <>
__device__ __forceinline__ void unpack16<__half>(const uint4& p, float (&f)[8]) {
    const uint32_t u[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = *reinterpret_cast<const __half2*>(&u[i]);
        float2 v = __half22float2(h);
        f[2 * i] = v.x;
        f[2 * i + 1] = v.y;
    }
}

template <>
__device__ __forceinline__ void unpack16<__nv_bfloat16>(const uint4& p, float (&f)[8]) {
    const uint32_t u[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(u[i] << 16);          // low half-word = even element
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

template <typename T> __device__ __forceinline__ uint4 pack16(const float (&f)[Elem<T>::kVec]);

template <>
__device__ __forceinline__ uint4 pack16<float>(const float (&f)[4]) {
    return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
}

template <>
__device__ __forceinline__ uint4 pack16<__half>(const float (&f)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
        u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(u[0], u[1], u[2], u[3]);
}

template <>
__device__ __forceinline__ uint4 pack16<__nv_bfloat16>(const float (&f)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
        u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return make_uint4(u[0], u[1], u[2], u[3]);
}

// Butterfly sum: every lane of the warp ends with the total (the order is fixed, so the result is
// bit-reproducible).
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v += __shfl_xor_sync(0xffffffffu, v, m);
    return v;
}

// Tells the compiler the packet may have changed. Used on loop-invariant packed operands (the weight
// row) at the top of a row loop so that their fp32 expansion is redone per row instead of being
// hoisted into 2-4x as many live registers.
__device__ __forceinline__ void keep_packed(uint4& p) {
    asm volatile("" : "+r"(p.x), "+r"(p.y), "+r"(p.z), "+r"(p.w));
}

// Asks L2 to fetch `bytes` (a multiple of 16) starting at a 16-byte aligned global address; nothing reaches the SM and
// no register is spent. The packet kernels issue it for the row a group will visit NEXT while they work on the
// current one: a thread holds one row's packets in registers, which limits what an SM has in flight to about 64 KB;
// with the next rows already on their way into L2 the following loads wait for L2 instead of HBM. Measured on B200
// (bf16, backward call, fraction of the copy bandwidth): hidden 8192 0.93 -> 1.00, hidden 16 384 0.85 -> 1.01,
// 8192 rows of hidden 8192 0.82 -> 0.88.
__device__ __forceinline__ void prefetch_l2_bulk(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// Streaming (read-once / write-once) 16-byte global accesses.
__device__ __forceinline__ uint4 ld_stream16(const uint4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream16(uint4* p, const uint4& v) { __stcs(p, v); }

}  // namespace mgr
