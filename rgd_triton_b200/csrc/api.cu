// Library-level entry points of librgd_b200: device check, status strings,
// launch accounting.
#include <atomic>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace rgd {

static std::atomic<int64_t> g_launches{0};

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_launch() { return cuda_status(cudaGetLastError()); }

int num_sms() {
    // Cached per device index; devices of one box are identical, but keep it exact.
    static std::atomic<int> cache[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cache[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

namespace {
struct LaunchKey {
    int dev;
    const void *kernel;
    uint64_t a, b;
    bool operator==(const LaunchKey &o) const { return dev == o.dev && kernel == o.kernel && a == o.a && b == o.b; }
};
struct LaunchKeyHash {
    size_t operator()(const LaunchKey &k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.kernel) * 0x9E3779B97F4A7C15ull;
        h ^= (k.a + 0x632BE59BD9B4E019ull) + (h << 6) + (h >> 2);
        h ^= (k.b + (uint64_t)k.dev * 0x100000001B3ull) + (h << 6) + (h >> 2);
        return (size_t)h;
    }
};
std::mutex g_launch_memo_mutex;
std::unordered_map<LaunchKey, int, LaunchKeyHash> g_smem_memo, g_occ_memo;
}  // namespace

int ensure_dyn_smem(const void *kernel, size_t bytes) {
    int dev = 0;
    if (cudaError_t e = cudaGetDevice(&dev); e != cudaSuccess) return cuda_status(e);
    const LaunchKey key{dev, kernel, (uint64_t)bytes, 0};
    {
        std::lock_guard<std::mutex> lock(g_launch_memo_mutex);
        auto it = g_smem_memo.find(key);
        if (it != g_smem_memo.end()) return it->second;
    }
    const int rc = cuda_status(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (rc != RGD_OK) {
        (void)cudaGetLastError();
        return rc;                      // not memoised: the next call asks the driver again
    }
    std::lock_guard<std::mutex> lock(g_launch_memo_mutex);
    g_smem_memo[key] = rc;
    return rc;
}

int cached_occupancy(const void *kernel, int threads, size_t smem) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    const LaunchKey key{dev, kernel, (uint64_t)threads, (uint64_t)smem};
    {
        std::lock_guard<std::mutex> lock(g_launch_memo_mutex);
        auto it = g_occ_memo.find(key);
        if (it != g_occ_memo.end()) return it->second;
    }
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem) != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        n = 1;
    }
    std::lock_guard<std::mutex> lock(g_launch_memo_mutex);
    g_occ_memo[key] = n;
    return n;
}

}  // namespace rgd

extern "C" int rgd_abi_version(void) { return 3; }

extern "C" int64_t rgd_launch_count(void) { return rgd::g_launches.load(std::memory_order_relaxed); }

extern "C" int rgd_device_supported(int device) {
    int major = 0;
    cudaError_t e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return RGD_E_DEVICE;
    }
    return major == 10 ? 1 : 0;
}

extern "C" const char *rgd_status_string(int status) {
    switch (status) {
        case RGD_OK: return "ok";
        case RGD_E_INVALID: return "invalid argument (shape mismatch or negative size)";
        case RGD_E_DTYPE: return "unsupported dtype for this operator";
        case RGD_E_SIZE: return "size outside the operator's limits";
        case RGD_E_STRIDE: return "stride or alignment the kernel cannot address";
        case RGD_E_NULL: return "required pointer is NULL";
        case RGD_E_WORKSPACE: return "workspace too small";
        case RGD_E_DEVICE: return "device is not compute capability 10.x (sm_100)";
        case RGD_E_BIAS_SHAPE: return "Last 2 dimensions of bias must be (1, seqlen_k) or (seqlen_q, seqlen_k)";
        case RGD_E_TIMEOUT: return "bounded device-side wait expired";
    }
    if (status >= RGD_E_CUDA_BASE && status < RGD_E_TIMEOUT)
        return cudaGetErrorString((cudaError_t)(status - RGD_E_CUDA_BASE));
    return "unknown status";
}
