// Micro-benchmark behind the structure of the tensor-memory attention kernels: how many clocks one
// tcgen05.mma (cta_group::1, kind::f16, M = 128, K = 16) takes, by shape of N, by where A comes
// from (shared memory: SS, tensor memory: TS), and by the number of issuing threads.  Every SM
// runs one CTA; a CTA's issuing thread(s) each issue `reps` groups of 8 MMAs back to back, commit
// to an mbarrier and wait for it with the library's bounded wait.  Prints clocks per MMA as seen
// by the first CTA.  A second kernel measures the CTA-pair form (cta_group::2, M = 256 over two
// SMs, each SM holding half of B's N rows), issued by one thread of the even CTA.
// Build and run: python -m rgd_triton_b200.microbench.run mma_rate
#include <cstdio>
#include <cuda_runtime.h>

#include "../csrc/sm100_prims.cuh"
using namespace rgd::sm100;

struct alignas(1024) Smem {
    unsigned char a[32768], b[65536];   // A: 128 x 128 16-bit, B: up to 256 x 128
    uint64_t done[4];
    uint32_t tmem_base;
};

// N: 64 / 128 / 256.  TS: A operand from tensor memory.  ISSUERS: 1, 2 or 4 issuing warps, each
// with its own accumulator columns.
template <int N, bool TS, int ISSUERS>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(int reps, long long *out, int *status) {
    extern __shared__ unsigned char raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    for (int i = threadIdx.x; i < (int)sizeof(sm.a) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(sm.a)[i] = 0x3c003c00u;
    for (int i = threadIdx.x; i < (int)sizeof(sm.b) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(sm.b)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(&sm.done[i], 1);
        fence_mbar_init();
    }
    if (threadIdx.x < 32) {
        tmem_alloc(&sm.tmem_base, 512);
        tmem_relinquish();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tb = sm.tmem_base;
    const int warp = threadIdx.x >> 5;
    if (warp < ISSUERS && (threadIdx.x & 31) == 0) {
        constexpr uint32_t idesc = make_idesc(true, 128, N, false, false);
        const uint64_t da = make_sdesc(smem_u32(sm.a), 16, 1024), db = make_sdesc(smem_u32(sm.b), 16, 1024);
        // accumulators of N columns per issuer; with N = 256 two issuers share nothing, four do not fit
        const uint32_t dcol = tb + (uint32_t)((warp * N) % 384);
        const long long t0 = clock64();
        for (int r = 0; r < reps; ++r) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                const uint32_t off = (kk / 4) * 16384 + (kk % 4) * 32;      // K-major, two 64-element panels
                if constexpr (TS) umma_ts(dcol, tb + 448 + kk * 8, sdesc_advance(db, off), idesc, true);
                else umma_ss(dcol, sdesc_advance(da, off), sdesc_advance(db, off), idesc, true);
            }
        }
        const long long t1 = clock64();
        umma_commit(&sm.done[warp]);
        const bool ok = mbar_wait(&sm.done[warp], 0, status, 7);
        const long long t2 = clock64();
        if (blockIdx.x == 0) {
            out[2 * warp] = t1 - t0;
            out[2 * warp + 1] = ok ? t2 - t0 : -1;
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) tmem_dealloc(tb, 512);
}

template <int N, bool TS, int ISSUERS>
static int run(const char *name, long long *out, int *status, int reps) {
    const size_t smem = sizeof(Smem) + 1024;
    cudaFuncSetAttribute(mma_rate_kernel<N, TS, ISSUERS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    mma_rate_kernel<N, TS, ISSUERS><<<148, 128, smem>>>(8, out, status);          // warm-up
    mma_rate_kernel<N, TS, ISSUERS><<<148, 128, smem>>>(reps, out, status);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h[8];
    int st = 0;
    cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
    cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    const double n = (double)reps * 8;
    printf("%-34s issue %6.1f clk/mma per thread, complete %6.1f clk/mma per thread, %5.1f clk/mma overall  (err %d, status %d)\n",
           name, h[0] / n, h[1] / n, h[1] / (n * ISSUERS), (int)e, st);
    return e != cudaSuccess || st != 0;
}

// CTA pair: M = 256 (128 rows per CTA), B's N rows split between the two CTAs.
template <int N, bool TS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) mma_rate_pair_kernel(int reps, long long *out, int *status) {
    extern __shared__ unsigned char raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    for (int i = threadIdx.x; i < (int)sizeof(sm.a) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(sm.a)[i] = 0x3c003c00u;
    for (int i = threadIdx.x; i < (int)sizeof(sm.b) / 4; i += blockDim.x) reinterpret_cast<uint32_t *>(sm.b)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) {
        mbar_init(&sm.done[0], 1);
        fence_mbar_init();
    }
    if (threadIdx.x < 32) {
        tmem_alloc_pair(&sm.tmem_base, 512);
        tmem_relinquish_pair();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before_sync();
    cluster_sync_all();
    tc_fence_after_sync();
    const uint32_t tb = sm.tmem_base;
    bool ok = true;
    if (threadIdx.x == 0) {
        long long t0 = 0, t1 = 0;
        if (cluster_ctarank() == 0) {
            constexpr uint32_t idesc = make_idesc(true, 256, N, false, false);
            const uint64_t da = make_sdesc(smem_u32(sm.a), 16, 1024), db = make_sdesc(smem_u32(sm.b), 16, 1024);
            t0 = clock64();
            for (int r = 0; r < reps; ++r) {
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // K-major operands, two 64-element panels: A panels of 128 rows, B panels of N / 2 rows
                    const uint32_t offa = (kk / 4) * 16384 + (kk % 4) * 32, offb = (kk / 4) * (N / 2 * 128) + (kk % 4) * 32;
                    if constexpr (TS) umma_ts_pair(tb, tb + 448 + kk * 8, sdesc_advance(db, offb), idesc, true);
                    else umma_ss_pair(tb, sdesc_advance(da, offa), sdesc_advance(db, offb), idesc, true);
                }
            }
            t1 = clock64();
            umma_commit_pair(&sm.done[0]);
        }
        ok = mbar_wait(&sm.done[0], 0, status, 8);      // both CTAs: the commit arrives in each
        const long long t2 = clock64();
        if (blockIdx.x == 0) {
            out[0] = t1 - t0;
            out[1] = ok ? t2 - t0 : -1;
        }
    }
    tc_fence_before_sync();
    cluster_sync_all();
    if (threadIdx.x < 32) tmem_dealloc_pair(tb, 512);
}

template <int N, bool TS>
static int run_pair(const char *name, long long *out, int *status, int reps) {
    const size_t smem = sizeof(Smem) + 1024;
    cudaFuncSetAttribute(mma_rate_pair_kernel<N, TS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    mma_rate_pair_kernel<N, TS><<<148, 128, smem>>>(8, out, status);
    mma_rate_pair_kernel<N, TS><<<148, 128, smem>>>(reps, out, status);
    const cudaError_t e = cudaDeviceSynchronize();
    long long h[2];
    int st = 0;
    cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
    cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost);
    const double n = (double)reps * 8;
    printf("%-34s issue %6.1f clk/mma, complete %6.1f clk/mma (256 rows over two SMs)  (err %d, status %d)\n", name, h[0] / n,
           h[1] / n, (int)e, st);
    return e != cudaSuccess || st != 0;
}

int main() {
    long long *out;
    int *status;
    cudaMalloc(&out, 64);
    cudaMalloc(&status, 4);
    cudaMemset(out, 0, 64);
    cudaMemset(status, 0, 4);
    const int reps = 2000;
    int bad = 0;
    bad |= run<256, false, 1>("SS N=256, 1 issuing thread", out, status, reps);
    bad |= run<128, false, 1>("SS N=128, 1 issuing thread", out, status, reps);
    bad |= run<128, true, 1>("TS N=128, 1 issuing thread", out, status, reps);
    bad |= run<64, false, 1>("SS N=64,  1 issuing thread", out, status, reps);
    bad |= run<64, true, 1>("TS N=64,  1 issuing thread", out, status, reps);
    bad |= run<128, false, 2>("SS N=128, 2 issuing threads", out, status, reps);
    bad |= run<64, false, 2>("SS N=64,  2 issuing threads", out, status, reps);
    bad |= run<64, false, 4>("SS N=64,  4 issuing threads", out, status, reps);
    bad |= run<64, true, 2>("TS N=64,  2 issuing threads", out, status, reps);
    bad |= run_pair<256, false>("pair SS N=256", out, status, reps);
    bad |= run_pair<128, false>("pair SS N=128", out, status, reps);
    bad |= run_pair<128, true>("pair TS N=128", out, status, reps);
    bad |= run_pair<64, false>("pair SS N=64", out, status, reps);
    printf(bad ? "FAILED\n" : "done\n");
    return bad;
}
