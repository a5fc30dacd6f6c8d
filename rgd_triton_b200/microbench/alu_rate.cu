// Micro-benchmark behind the softmax of the attention forward: results per clock per SM of the
// instructions its inner loop is made of, each alone and in the loop's own mix, with 8 warps per
// SM (two per scheduler, as in the kernel).  ex2 = ex2.approx.ftz.f32; pack = cvt.rn.bf16x2.f32
// (two values per instruction); fma = fma.rn.f32; ipack = the 16-bit pack done with integer
// instructions (add 0x8000, byte permute).  Every thread runs 8 independent chains.
// Build and run: python -m rgd_triton_b200.microbench.run alu_rate
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

template <int MODE>
__global__ void __launch_bounds__(256, 1) alu_rate_kernel(int reps, float seed, long long *out, float *sink) {
    float x[8];
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) x[i] = seed + 0.001f * (float)(threadIdx.x + 32 * i);
    __syncthreads();
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            float a = x[i], b = x[i + 1];
            if (MODE == 0 || MODE == 4 || MODE == 5) {                    // ex2
                asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(a));
                asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(b));
            }
            if (MODE == 1 || MODE == 4) {                                 // pack by cvt
                uint32_t pk;
                asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk) : "f"(b), "f"(a));
                acc ^= pk;
            }
            if (MODE == 2) {                                              // fma
                asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(a) : "f"(seed));
                asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(b) : "f"(seed));
            }
            if (MODE == 3 || MODE == 5) {                                 // pack by integer instructions
                const uint32_t ua = __float_as_uint(a) + 0x8000u, ub = __float_as_uint(b) + 0x8000u;
                uint32_t pk;
                asm volatile("prmt.b32 %0, %1, %2, 0x7632;" : "=r"(pk) : "r"(ua), "r"(ub));
                acc ^= pk;
            }
            if (MODE == 4 || MODE == 5) {                                 // the rest of the loop's mix: scale, row sum
                asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(a) : "f"(seed));
                asm volatile("fma.rn.f32 %0, %0, %1, %1;" : "+f"(b) : "f"(seed));
                asm volatile("add.f32 %0, %0, %1;" : "+f"(a) : "f"(b));
            }
            if (MODE == 6 || MODE == 7) {                                 // packed 16-bit ex2: two values per instruction
                uint32_t pk;
                if (MODE == 6) {
                    asm volatile("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(pk) : "f"(b), "f"(a));
                    asm volatile("ex2.approx.ftz.bf16x2 %0, %0;" : "+r"(pk));
                } else {
                    asm volatile("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(pk) : "f"(b), "f"(a));
                    asm volatile("ex2.approx.f16x2 %0, %0;" : "+r"(pk));
                }
                acc ^= pk;
                a = __uint_as_float((pk << 16) | 0x3c000000u) - 1.0f;      // keep the chain dependent on the result
                b = __uint_as_float((pk & 0xffff0000u) | 0x3c00u) - 1.0f;
            }
            x[i] = a;
            x[i + 1] = b;
        }
    }
    const long long t1 = clock64();
    float s = __uint_as_float(acc & 0x3fffffffu);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += x[i];
    if (s == 12345.678f) sink[0] = s;
    if (blockIdx.x == 0 && threadIdx.x == 0) out[0] = t1 - t0;
}

template <int MODE>
static void run(const char *name, double per_iter, long long *out, float *sink) {
    const int reps = 4096;
    alu_rate_kernel<MODE><<<148, 256>>>(16, 0.5f, out, sink);
    alu_rate_kernel<MODE><<<148, 256>>>(reps, 0.5f, out, sink);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h = 0;
    cudaMemcpy(&h, out, sizeof(h), cudaMemcpyDeviceToHost);
    // per repetition a thread handles 8 values; 256 threads per SM
    printf("%-44s %7.1f clk per 8 values per thread -> %6.1f values / clk / SM (%s per value)  (err %d)\n", name,
           (double)h / reps, 8.0 * 256.0 * reps / (double)h, per_iter == 0.5 ? "half an instruction" : "one instruction", (int)e);
}

int main() {
    long long *out;
    float *sink;
    cudaMalloc(&out, 8);
    cudaMalloc(&sink, 4);
    run<0>("ex2.approx.ftz.f32", 1, out, sink);
    run<1>("cvt.rn.bf16x2.f32 (pack)", 0.5, out, sink);
    run<2>("fma.rn.f32", 1, out, sink);
    run<3>("integer pack (add + prmt)", 1, out, sink);
    run<4>("loop mix: fma, ex2, add, cvt pack", 1, out, sink);
    run<5>("loop mix: fma, ex2, add, integer pack", 1, out, sink);
    run<6>("cvt pack + ex2.approx.ftz.bf16x2 + unpack", 1, out, sink);
    run<7>("cvt pack + ex2.approx.f16x2 + unpack", 1, out, sink);
    printf("done\n");
    return 0;
}
