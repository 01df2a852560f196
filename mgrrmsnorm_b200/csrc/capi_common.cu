// Entry points of libmgr_b200.so that are not tied to one kernel family: version, status names,
// device probe.

#include <atomic>
#include <cstdlib>
#include <cstring>

#include "mgr_common.cuh"

namespace mgr {

namespace {
std::atomic<bool> g_env_loaded{false};
std::atomic<int> g_env[8];

void load_env() {
    auto num = [](const char* name, int unset) {
        const char* e = std::getenv(name);
        return (e == nullptr || e[0] == '\0') ? unset : std::atoi(e);
    };
    int path = 0;
    if (const char* e = std::getenv("MGR_RMSNORM_PATH")) {
        if (std::strcmp(e, "reg") == 0) path = 1;
        else if (std::strcmp(e, "ring") == 0) path = 2;
        else if (std::strcmp(e, "scalar") == 0) path = 3;
    }
    int cg = 0;
    if (const char* e = std::getenv("MGR_GEMM_CTA_GROUP")) cg = e[0] == '2' ? 2 : (e[0] == '1' ? 1 : 0);
    int pdl = 1;
    if (const char* e = std::getenv("MGR_GEMM_PDL")) pdl = e[0] != '0';
    int narrow = -1;
    if (const char* e = std::getenv("MGR_GEMM_NARROW")) narrow = e[0] == '0' ? 0 : (e[0] == '3' ? 32 : (e[0] == '9' ? 96 : 64));
    g_env[0].store(path, std::memory_order_relaxed);
    g_env[1].store(num("MGR_RMSNORM_FWD_SHAPE", -1), std::memory_order_relaxed);
    g_env[2].store(num("MGR_RMSNORM_BWD_SHAPE", -1), std::memory_order_relaxed);
    g_env[3].store(num("MGR_RMSNORM_BWD_FAT", -1), std::memory_order_relaxed);
    g_env[4].store(cg, std::memory_order_relaxed);
    g_env[5].store(pdl, std::memory_order_relaxed);
    g_env[6].store(narrow, std::memory_order_relaxed);
    g_env[7].store(num("MGR_RMSNORM_PREFETCH", -1), std::memory_order_relaxed);
    g_env_loaded.store(true, std::memory_order_release);
}
}  // namespace

Overrides overrides() {
    if (!g_env_loaded.load(std::memory_order_acquire)) load_env();   // racing first calls read the same environment
    Overrides o;
    o.rms_path = g_env[0].load(std::memory_order_relaxed);
    o.fwd_shape = g_env[1].load(std::memory_order_relaxed);
    o.bwd_shape = g_env[2].load(std::memory_order_relaxed);
    o.bwd_fat = g_env[3].load(std::memory_order_relaxed);
    o.cta_group = g_env[4].load(std::memory_order_relaxed);
    o.pdl = g_env[5].load(std::memory_order_relaxed);
    o.narrow = g_env[6].load(std::memory_order_relaxed);
    o.prefetch = g_env[7].load(std::memory_order_relaxed);
    return o;
}

DeviceInfo current_device_info() {
    // Filled once per device; `known` is published with release order after the entry is complete, so a thread
    // that sees it set reads a whole entry. Two threads racing on the first call both write the same values.
    static DeviceInfo cache[kMaxDevices];
    static std::atomic<bool> known[kMaxDevices];
    DeviceInfo di{MGR_ERR_CUDA, -1, 0};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        (void)cudaGetLastError();
        return di;
    }
    if (known[dev].load(std::memory_order_acquire)) return cache[dev];
    int major = 0, sms = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return di;
    }
    di.device = dev;
    di.sm_count = sms;
    di.status = (major == 10) ? MGR_OK : MGR_ERR_UNSUPPORTED_ARCH;
    cache[dev] = di;
    known[dev].store(true, std::memory_order_release);
    return di;
}

int rmsnorm_status_fetch(int clear);  // rmsnorm_sm100.cu
int gemm_status_fetch(int clear);     // gemm_sm100.cu
int peer_status_fetch(int clear);     // peer_allreduce_sm100.cu
int rmsnorm_status_poke(int value);   // rmsnorm_sm100.cu
int gemm_status_poke(int value);      // gemm_sm100.cu

}  // namespace mgr

extern "C" int mgr_device_status(int clear) {
    const mgr::DeviceInfo di = mgr::current_device_info();
    if (di.status != MGR_OK) return di.status;
    const int a = mgr::rmsnorm_status_fetch(clear);
    const int b = mgr::gemm_status_fetch(clear);
    const int c = mgr::peer_status_fetch(clear);
    return a != MGR_OK ? a : (b != MGR_OK ? b : c);
}

extern "C" int mgr_debug_poke_device_status(int family, int value) {
    const mgr::DeviceInfo di = mgr::current_device_info();
    if (di.status != MGR_OK) return di.status;
    if (family == 0) return mgr::rmsnorm_status_poke(value);
    if (family == 1) return mgr::gemm_status_poke(value);
    return MGR_ERR_BAD_SHAPE;
}

extern "C" void mgr_reload_env(void) { mgr::load_env(); }

extern "C" int mgr_abi_version(void) { return MGR_ABI_VERSION; }

extern "C" const char* mgr_status_str(int status) {
    switch (status) {
        case MGR_OK: return "ok";
        case MGR_ERR_BAD_DTYPE: return "unsupported dtype (use MGR_F32, MGR_F16 or MGR_BF16)";
        case MGR_ERR_BAD_SHAPE: return "bad shape (negative rows, non-positive cols or inconsistent dimensions)";
        case MGR_ERR_NULL_PTR: return "required pointer is NULL";
        case MGR_ERR_MISALIGNED: return "pointer is not aligned to its element size (workspace: 16 bytes)";
        case MGR_ERR_WORKSPACE_TOO_SMALL: return "workspace is smaller than the size the *_workspace_bytes query returns";
        case MGR_ERR_UNSUPPORTED_ARCH: return "current device is not compute capability 10.x (library is sm_100a only)";
        case MGR_ERR_LAUNCH_FAILED: return "kernel launch failed";
        case MGR_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case MGR_ERR_TOO_LARGE: return "dimension exceeds the supported maximum";
        case MGR_ERR_CUDA: return "CUDA runtime call failed (no usable device?)";
        default: return "unknown status";
    }
}

extern "C" int mgr_device_check(int* sm_count) {
    const mgr::DeviceInfo di = mgr::current_device_info();
    if (sm_count != nullptr) *sm_count = di.sm_count;
    return di.status;
}
