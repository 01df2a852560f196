// Cross-rank sum of a short fp32 vector (the dW of a row-sharded RMSNorm: [H] floats, 32 KB at H = 8192) over
// NVLink peer memory, one process per GPU.
//
// The reference has no distributed code. The library's multi-GPU layer first summed dW with an NCCL all-reduce, which
// for 32 KB is pure latency: 18 us on 2-4 GPUs and 55 us on 8, against a rank's whole forward+backward of about
// 105 us once 65 536 rows are split eight ways. This kernel is the same sum as ONE launch per rank over memory every
// rank can write (torch symmetric memory; any peer-mapped allocation will do):
//   1. every CTA owns a slice of the vector; it stores this rank's slice into slot [rank] of EVERY rank's buffer
//      (plain peer stores: posted writes, no round trip), fences, and raises its flag in every rank's flag array;
//   2. it waits (bounded) until every rank's flag for this slice has arrived in its own flag array;
//   3. it adds the P slots of its slice in rank order and writes the fp32 sum and its one rounding to the weight type.
// The order of the additions is the rank order on every rank, so all ranks hold the same bits, and the same bits as a
// one-rank run that adds the partials in that order. CTAs never wait for other CTAs of the same GPU, only for the
// same slice on other GPUs, so no grid-wide barrier and no co-residency requirement on one GPU arises. Buffers are
// double-buffered by the parity of a per-CTA call counter kept in device memory (so a captured graph replays
// correctly): a rank can be at most one call ahead of any other, because finishing call k needs every rank's flag k.
// No multicast and no remote loads are involved: stores to peers, loads from local memory.

#include <atomic>

#include "mgr_common.cuh"

namespace mgr {
namespace {

__device__ int g_peer_status = 0;

constexpr int kPeerMaxRanks = 16;
constexpr int kPeerThreads = 256;

struct PeerBufs {
    unsigned char* base[kPeerMaxRanks];   // rank q's buffer, as mapped in THIS process
};

// Byte layout of every rank's buffer for vectors of up to `n_max` floats and `world` ranks:
//   [0, 2 * world * n_max * 4)                 data: [parity][sender][n_max] floats
//   [flags_off, + world * kPeerCtas * 4)       flags: [sender][cta] call numbers
__host__ __device__ inline size_t peer_flags_offset(int world, int64_t n_max) {
    return (static_cast<size_t>(2) * world * n_max * 4 + 255) / 256 * 256;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <typename T>
__global__ void __launch_bounds__(kPeerThreads)
peer_allreduce_f32(PeerBufs bufs, int rank, int world, const float* __restrict__ src, float* __restrict__ out_f32,
                   T* __restrict__ out_t, int n, int64_t n_max, uint32_t* __restrict__ calls /* [gridDim.x], local */,
                   int* __restrict__ status) {
    __shared__ uint32_t call_s;
    __shared__ int abort_s;
    const int cta = blockIdx.x, ctas = gridDim.x;
    if (threadIdx.x == 0) {
        call_s = calls[cta] + 1;
        abort_s = 0;
    }
    __syncthreads();
    const uint32_t call = call_s;
    const int parity = static_cast<int>(call & 1u);
    const size_t flags_off = peer_flags_offset(world, n_max);
    // this CTA's slice, in packets of four floats (n is a multiple of 4)
    const int n4 = n >> 2;
    const int per = (n4 + ctas - 1) / ctas;
    const int lo = cta * per, hi = lo + per < n4 ? lo + per : n4;

    // 1. this rank's slice into slot [rank] of every rank's buffer
    const float4* s4 = reinterpret_cast<const float4*>(src);
    for (int q = 0; q < world; ++q) {
        float4* dst = reinterpret_cast<float4*>(bufs.base[q]) + (static_cast<size_t>(parity) * world + rank) * (n_max >> 2);
        for (int i = lo + threadIdx.x; i < hi; i += kPeerThreads) dst[i] = s4[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
        uint32_t* flag = reinterpret_cast<uint32_t*>(bufs.base[threadIdx.x] + flags_off) + static_cast<size_t>(rank) * ctas + cta;
        st_release_sys(flag, call);
    }

    // 2. every rank's slice has arrived here (bounded wait: about a second, then the status word says so)
    if (threadIdx.x < world) {
        const uint32_t* flag = reinterpret_cast<const uint32_t*>(bufs.base[rank] + flags_off) + static_cast<size_t>(threadIdx.x) * ctas + cta;
        bool seen = false;
        for (int spin = 0; spin < (1 << 22); ++spin) {
            if (static_cast<int32_t>(ld_acquire_sys(flag) - call) >= 0) {
                seen = true;
                break;
            }
            __nanosleep(200);
        }
        if (!seen) abort_s = 1;
    }
    __syncthreads();
    if (abort_s != 0) {
        if (threadIdx.x == 0) {
            atomicExch(status, MGR_ERR_DEVICE_TIMEOUT);
            calls[cta] = call;
        }
        return;
    }

    // 3. the sum, in rank order, from local memory (written by the peers: read past L1)
    const float4* mine = reinterpret_cast<const float4*>(bufs.base[rank]) + static_cast<size_t>(parity) * world * (n_max >> 2);
    for (int i = lo + threadIdx.x; i < hi; i += kPeerThreads) {
        float4 a = __ldcg(mine + i);
        for (int q = 1; q < world; ++q) {
            const float4 b = __ldcg(mine + static_cast<size_t>(q) * (n_max >> 2) + i);
            a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
        }
        if (out_f32 != nullptr) reinterpret_cast<float4*>(out_f32)[i] = a;
        if (out_t != nullptr) {
            out_t[4 * i] = from_f32<T>(a.x);
            out_t[4 * i + 1] = from_f32<T>(a.y);
            out_t[4 * i + 2] = from_f32<T>(a.z);
            out_t[4 * i + 3] = from_f32<T>(a.w);
        }
    }
    if (threadIdx.x == 0) calls[cta] = call;
}

int* peer_status_ptr(const DeviceInfo& di) {
    static std::atomic<int*> cache[kMaxDevices];
    if (cache[di.device].load(std::memory_order_relaxed) == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_peer_status) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        cache[di.device].store(static_cast<int*>(p), std::memory_order_relaxed);
    }
    return cache[di.device].load(std::memory_order_relaxed);
}

}  // namespace

int peer_status_fetch(int clear) {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_peer_status, sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        return MGR_ERR_CUDA;
    }
    if (clear && v != 0) {
        const int zero = 0;
        if (cudaMemcpyToSymbol(g_peer_status, &zero, sizeof(int)) != cudaSuccess) (void)cudaGetLastError();
    }
    return v;
}

}  // namespace mgr

using namespace mgr;

extern "C" size_t mgr_peer_allreduce_buffer_bytes(int world, int64_t n_max) {
    if (world < 1 || world > kPeerMaxRanks || n_max < 4 || n_max % 4 != 0 || n_max > (1ll << 24)) return 0;
    return peer_flags_offset(world, n_max) + static_cast<size_t>(world) * MGR_PEER_ALLREDUCE_CTAS * 4;
}

extern "C" int mgr_peer_allreduce_f32(const void* const* peer_buffers, int rank, int world, const float* src, float* out_f32,
                                      void* out, int dtype, int64_t n, int64_t n_max, void* calls, void* stream) {
    if (dtype_size(dtype) == 0) return MGR_ERR_BAD_DTYPE;
    if (world < 1 || world > kPeerMaxRanks || rank < 0 || rank >= world) return MGR_ERR_BAD_SHAPE;
    if (n < 4 || n % 4 != 0 || n_max < n || n_max % 4 != 0 || n_max > (1ll << 24)) return MGR_ERR_BAD_SHAPE;
    if (peer_buffers == nullptr || src == nullptr || calls == nullptr || (out_f32 == nullptr && out == nullptr)) return MGR_ERR_NULL_PTR;
    if (!aligned_to(src, 16) || !aligned_to(out_f32, 16) || !aligned_to(out, dtype_size(dtype)) || !aligned_to(calls, 4)) return MGR_ERR_MISALIGNED;
    PeerBufs bufs{};
    for (int q = 0; q < world; ++q) {
        if (peer_buffers[q] == nullptr) return MGR_ERR_NULL_PTR;
        if (!aligned_to(peer_buffers[q], 256)) return MGR_ERR_MISALIGNED;
        bufs.base[q] = static_cast<unsigned char*>(const_cast<void*>(peer_buffers[q]));
    }
    const DeviceInfo di = current_device_info();
    if (di.status != MGR_OK) return di.status;
    int* status = peer_status_ptr(di);
    if (status == nullptr) return MGR_ERR_CUDA;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int nn = static_cast<int>(n);
    uint32_t* c = static_cast<uint32_t*>(calls);
    switch (dtype) {
        case MGR_F32:
            peer_allreduce_f32<float><<<MGR_PEER_ALLREDUCE_CTAS, kPeerThreads, 0, s>>>(bufs, rank, world, src, out_f32, static_cast<float*>(out), nn, n_max, c, status);
            break;
        case MGR_F16:
            peer_allreduce_f32<__half><<<MGR_PEER_ALLREDUCE_CTAS, kPeerThreads, 0, s>>>(bufs, rank, world, src, out_f32, static_cast<__half*>(out), nn, n_max, c, status);
            break;
        default:
            peer_allreduce_f32<__nv_bfloat16><<<MGR_PEER_ALLREDUCE_CTAS, kPeerThreads, 0, s>>>(bufs, rank, world, src, out_f32, static_cast<__nv_bfloat16*>(out), nn, n_max, c, status);
            break;
    }
    return launch_status();
}
