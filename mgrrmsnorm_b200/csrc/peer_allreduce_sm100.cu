// Cross-rank sum of a short fp32 vector (the dW of a row-sharded RMSNorm: [H] floats, 32 KB at H = 8192) over
// NVLink peer memory, one process per GPU.
//
// The reference has no distributed code. The library's multi-GPU layer first summed dW with an NCCL all-reduce, which
// for 32 KB is pure latency: 18 us on 2-4 GPUs and 26-55 us on 8, against a rank's whole forward+backward of about
// 105 us once 65 536 rows are split eight ways. This kernel is the same sum as ONE launch per rank over memory every
// rank can write (torch symmetric memory; any peer-mapped allocation will do):
//   1. every CTA owns a slice of the vector; it stores this rank's slice into slot [rank] of EVERY rank's buffer, each
//      value paired with the number of this call in one 8-byte store (plain peer stores: posted writes, no round trip);
//   2. it reads the P slots of its slice from its OWN buffer, waiting (bounded) on each element until it carries this
//      call's number, adds them in rank order and writes the fp32 sum and its one rounding to the weight type.
// The order of the additions is the rank order on every rank, so all ranks hold the same bits, and the same bits as a
// one-rank run that adds the partials in that order. CTAs never wait for other CTAs of the same GPU, only for the
// same elements from other GPUs, so no grid-wide barrier and no co-residency requirement on one GPU arises. Buffers
// are double-buffered by the parity of a per-CTA call counter kept in device memory (so a captured graph replays
// correctly): a rank can be at most one call ahead of any other, because finishing call k needs every rank's
// elements of call k, and those are only written once that rank has finished reading call k - 1.
// No multicast, no fences and no remote loads are involved: 8-byte stores to peers, 8-byte loads from local memory.

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
//   [parity][sender][n_max] pairs {float bits, call number}, 8 bytes each
// A pair is written with ONE 8-byte store and read with ONE 8-byte load, which are single accesses on NVLink as on
// local memory: whoever sees the call number of this call sees the value written with it. So no fence and no
// separate flag are needed (the fence.sys + release / acquire form of this kernel took 13 us on ONE rank; this form
// takes 3), and a reader only ever waits for the very elements it is about to add.
__host__ __device__ inline size_t peer_buffer_bytes(int world, int64_t n_max) {
    return static_cast<size_t>(2) * world * n_max * 8;
}

__device__ __forceinline__ void st_pair(uint2* p, uint32_t value, uint32_t call) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(value), "r"(call) : "memory");
}
__device__ __forceinline__ uint2 ld_pair(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
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
    const size_t parity = call & 1u;
    // this CTA's slice of the vector
    const int per = (n + ctas - 1) / ctas;
    const int lo = cta * per, hi = lo + per < n ? lo + per : n;

    // 1. this rank's slice, paired with the call number, into slot [rank] of every rank's buffer (peer stores)
    for (int i = lo + threadIdx.x; i < hi; i += kPeerThreads) {
        const uint32_t v = __float_as_uint(src[i]);
        for (int q = 0; q < world; ++q) {
            uint2* dst = reinterpret_cast<uint2*>(bufs.base[q]) + (parity * world + rank) * n_max;
            st_pair(dst + i, v, call);
        }
    }

    // 2. + 3. every rank's element as it arrives here (bounded wait: about a second in all, then the status word
    // says so), added in rank order from local memory
    const uint2* mine = reinterpret_cast<const uint2*>(bufs.base[rank]) + parity * world * n_max;
    bool ok = true;
    int budget = 1 << 22;
    for (int i = lo + threadIdx.x; i < hi && ok; i += kPeerThreads) {
        float sum = 0.f;
        for (int q = 0; q < world && ok; ++q) {
            const uint2* p = mine + static_cast<size_t>(q) * n_max + i;
            uint2 v = ld_pair(p);
            while (v.y != call) {
                if (--budget <= 0 || *reinterpret_cast<volatile int*>(&abort_s) != 0) {
                    ok = false;
                    break;
                }
                __nanosleep(100);
                v = ld_pair(p);
            }
            sum = q == 0 ? __uint_as_float(v.x) : sum + __uint_as_float(v.x);
        }
        if (ok) {
            if (out_f32 != nullptr) out_f32[i] = sum;
            if (out_t != nullptr) out_t[i] = from_f32<T>(sum);
        }
    }
    if (!ok) abort_s = 1;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (abort_s != 0) atomicExch(status, MGR_ERR_DEVICE_TIMEOUT);
        calls[cta] = call;
    }
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
    return peer_buffer_bytes(world, n_max);
}

extern "C" int mgr_peer_allreduce_f32(const void* const* peer_buffers, int rank, int world, const float* src, float* out_f32,
                                      void* out, int dtype, int64_t n, int64_t n_max, void* calls, void* stream) {
    if (dtype_size(dtype) == 0) return MGR_ERR_BAD_DTYPE;
    if (world < 1 || world > kPeerMaxRanks || rank < 0 || rank >= world) return MGR_ERR_BAD_SHAPE;
    if (n < 4 || n % 4 != 0 || n_max < n || n_max % 4 != 0 || n_max > (1ll << 24)) return MGR_ERR_BAD_SHAPE;   // (multiples of 4: 16-byte rows)
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
