// Micro-benchmark: throughput of fp32 reductions into global memory that is resident in L2 (or
// not), the quantity that bounds a single-pass attention backward which adds its dQ partial
// tiles into an fp32 accumulator.  Forms: 16-byte vector reductions (a warp covers 512 contiguous
// bytes), four coalesced scalar reductions, bulk reductions from shared memory, and plain 16-byte
// stores as the yardstick.  Bounded loops only.
// Build and run: python -m rgd_triton_b200.microbench.run l2_reduction
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#define CK(x)                                                                    \
    do {                                                                         \
        cudaError_t e_ = (x);                                                    \
        if (e_ != cudaSuccess) {                                                 \
            printf("error %s at line %d\n", cudaGetErrorString(e_), __LINE__);   \
            return 1;                                                            \
        }                                                                        \
    } while (0)

// MODE 0: red.global.add.v4.f32; 1: st.global.v4.f32; 2: four scalar red.global.add.f32, each coalesced
template <int MODE>
__global__ void __launch_bounds__(256) reduce_kernel(float *buf, size_t region_f4, int iters) {
    const size_t stride = (size_t)gridDim.x * 256;
    size_t idx = ((size_t)blockIdx.x * 256 + threadIdx.x) % region_f4;
    const float a = 1.f, b = 2.f, c = 3.f, d = 4.f;
    for (int i = 0; i < iters; ++i) {
        float *p = buf + idx * 4;
        if (MODE == 0) {
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
        } else if (MODE == 1) {
            asm volatile("st.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
        } else {
            float *q = buf + (idx - threadIdx.x % 32) * 4 + threadIdx.x % 32;
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(q), "f"(a) : "memory");
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(q + 32), "f"(b) : "memory");
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(q + 64), "f"(c) : "memory");
            asm volatile("red.global.add.f32 [%0], %1;" ::"l"(q + 96), "f"(d) : "memory");
        }
        idx += stride;
        if (idx >= region_f4) idx -= region_f4;
    }
}

// One thread per CTA adds `chunk` bytes of shared memory per iteration with a bulk reduction.
__global__ void __launch_bounds__(128) bulk_reduce_kernel(float *buf, size_t region_bytes, int iters, int chunk) {
    extern __shared__ __align__(128) unsigned char sm[];
    for (int i = threadIdx.x; i < chunk / 4; i += blockDim.x) reinterpret_cast<float *>(sm)[i] = 1.f;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    if (threadIdx.x == 0) {
        size_t off = ((size_t)blockIdx.x * chunk) % region_bytes;
        const uint32_t s = (uint32_t)__cvta_generic_to_shared(sm);
        for (int i = 0; i < iters; ++i) {
            asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(
                             reinterpret_cast<char *>(buf) + off),
                         "r"(s), "r"(chunk)
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 4;" ::: "memory");
            off += (size_t)gridDim.x * chunk;
            if (off >= region_bytes) off -= region_bytes;
        }
        asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    }
}

int main() {
    float *buf;
    const size_t cap = 256u << 20;
    CK(cudaMalloc(&buf, cap));
    CK(cudaMemset(buf, 0, cap));
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const int iters = 2000, ctas = 148 * 8;
    const char *names[3] = {"red.global.add.v4.f32", "st.global.v4.f32 (yardstick)", "red.global.add.f32 x 4"};
    for (size_t region_mb : {8, 32, 128}) {
        const size_t region_f4 = (region_mb << 20) / 16;
        for (int mode = 0; mode < 3; ++mode) {
            float best = 1e9f;
            for (int rep = 0; rep < 3; ++rep) {
                CK(cudaEventRecord(e0));
                if (mode == 0) reduce_kernel<0><<<ctas, 256>>>(buf, region_f4, iters);
                else if (mode == 1) reduce_kernel<1><<<ctas, 256>>>(buf, region_f4, iters);
                else reduce_kernel<2><<<ctas, 256>>>(buf, region_f4, iters);
                CK(cudaEventRecord(e1));
                CK(cudaEventSynchronize(e1));
                float ms;
                cudaEventElapsedTime(&ms, e0, e1);
                best = ms < best ? ms : best;
            }
            printf("target %3zu MB  %-30s %8.1f GB/s\n", region_mb, names[mode], (double)ctas * 256 * 16 * iters / best / 1e6);
        }
        const int chunk = 16384, bctas = 296, it2 = 400;
        CK(cudaFuncSetAttribute(bulk_reduce_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 65536));
        float best = 1e9f;
        for (int rep = 0; rep < 3; ++rep) {
            CK(cudaEventRecord(e0));
            bulk_reduce_kernel<<<bctas, 128, chunk>>>(buf, region_mb << 20, it2, chunk);
            CK(cudaEventRecord(e1));
            CK(cudaEventSynchronize(e1));
            float ms;
            cudaEventElapsedTime(&ms, e0, e1);
            best = ms < best ? ms : best;
        }
        printf("target %3zu MB  %-30s %8.1f GB/s\n", region_mb, "cp.reduce.async.bulk add.f32 16 KB", (double)bctas * chunk * it2 / best / 1e6);
    }
    CK(cudaDeviceSynchronize());
    printf("done\n");
    return 0;
}
