// Shared device/host helpers for the sm_100a kernels of librgd_b200.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/rgd_b200.h"

namespace rgd {

// ---------------------------------------------------------------------------
// Launch bookkeeping
// ---------------------------------------------------------------------------
void count_launch();                    // defined in api.cu
int  check_launch();                    // cudaGetLastError -> status code
int  num_sms();                         // SM count of the current device (cached)
// Opt a kernel in to `bytes` of dynamic shared memory.  The driver call is made once per
// (device, kernel, size); later launches only look the answer up.
int  ensure_dyn_smem(const void *kernel, size_t bytes);
// cudaOccupancyMaxActiveBlocksPerMultiprocessor, memoised per (device, kernel, threads,
// shared memory).  Never returns less than 1.
int  cached_occupancy(const void *kernel, int threads, size_t smem);

static inline int cuda_status(cudaError_t e) {
    return e == cudaSuccess ? RGD_OK : RGD_E_CUDA_BASE + (int)e;
}

// ---------------------------------------------------------------------------
// Scalar conversions
// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Round a float to the precision of T and come back (one RTNE rounding).
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32<T>(from_f32<T>(v)); }

// ---------------------------------------------------------------------------
// Fixed-width register vectors: N elements of T moved with one access when
// N * sizeof(T) is 16 bytes (or 8 / 4 for the narrower cases).
// ---------------------------------------------------------------------------
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
    T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_vec(const T *p) {
    return *reinterpret_cast<const Vec<T, N> *>(p);
}
template <typename T, int N>
__device__ __forceinline__ void store_vec(T *p, const Vec<T, N> &v) {
    *reinterpret_cast<Vec<T, N> *>(p) = v;
}

// Streaming (evict-first) 16-byte accesses for data touched exactly once.
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 r;
    asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st_stream16(void *p, const uint4 &v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

// Vector accesses with the evict-first hint when the vector is 16 bytes wide.
template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_vec_stream(const T *p) {
    if constexpr (sizeof(T) * N == 16) {
        union { uint4 u; Vec<T, N> v; } c;
        c.u = ld_stream16(p);
        return c.v;
    } else {
        return load_vec<T, N>(p);
    }
}
template <typename T, int N>
__device__ __forceinline__ void store_vec_stream(T *p, const Vec<T, N> &v) {
    if constexpr (sizeof(T) * N == 16) {
        union { uint4 u; Vec<T, N> v; } c;
        c.v = v;
        st_stream16(p, c.u);
    } else {
        store_vec<T, N>(p, v);
    }
}

// Elements of T per 16-byte access.
template <typename T> struct VecElems { static constexpr int value = 16 / sizeof(T); };

template <typename T> struct DTypeCode;
template <> struct DTypeCode<float> { static constexpr int value = RGD_F32; };
template <> struct DTypeCode<__half> { static constexpr int value = RGD_F16; };
template <> struct DTypeCode<__nv_bfloat16> { static constexpr int value = RGD_BF16; };

static inline int dtype_size(int dt) { return dt == RGD_F32 ? 4 : 2; }
static inline bool dtype_ok(int dt) { return dt == RGD_F32 || dt == RGD_F16 || dt == RGD_BF16; }

// Load one element of runtime dtype as fp32 (weights, tables: small, cached).
__device__ __forceinline__ float load_as_f32(const void *base, int64_t idx, int dt) {
    if (dt == RGD_F32) return reinterpret_cast<const float *>(base)[idx];
    if (dt == RGD_F16) return __half2float(reinterpret_cast<const __half *>(base)[idx]);
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(base)[idx]);
}
__device__ __forceinline__ void store_from_f32(void *base, int64_t idx, int dt, float v) {
    if (dt == RGD_F32) reinterpret_cast<float *>(base)[idx] = v;
    else if (dt == RGD_F16) reinterpret_cast<__half *>(base)[idx] = __float2half_rn(v);
    else reinterpret_cast<__nv_bfloat16 *>(base)[idx] = __float2bfloat16_rn(v);
}

// ---------------------------------------------------------------------------
// Reductions over a power-of-two group of `width` consecutive threads.
// width <= 32: xor shuffles.  width > 32: shuffles + one shared-memory hop
// (all threads of the CTA must call; `scratch` holds >= 2 * 8 floats... see use).
// ---------------------------------------------------------------------------
__device__ __forceinline__ float warp_group_sum(float v, int width) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        if (o < width) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

static inline bool is_aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

static inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline int next_pow2(int v) {
    int p = 1;
    while (p < v) p <<= 1;
    return p;
}

}  // namespace rgd
