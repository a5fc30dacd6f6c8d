// Library-level entry points of librgd_b200: device check, status strings,
// launch accounting.
#include <atomic>

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

}  // namespace rgd

extern "C" int rgd_abi_version(void) { return 1; }

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
