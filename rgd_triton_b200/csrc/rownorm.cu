// Row normalisations over [B, N, C] tensors: L2 normalise and RMS norm with an
// affine weight, forward and backward, for one or two tensors per launch.
//
// Bandwidth-bound design: a group of `tpr` consecutive threads owns one row and
// keeps it in registers (one 16-byte access per thread and per column slot, so
// every tensor is read exactly once and written exactly once), row sums are
// reduced with shuffles (plus one shared-memory hop when a row spans several
// warps), and all arithmetic is fp32.  A CTA walks the rows of one batch of one
// tensor; with two tensors the block index selects the tensor, which is the
// reference's "virtual tensor" fusion (fused_rmsnorm_cached.py:429).
//
// dweight is accumulated per thread over all rows the CTA visits, reduced over
// the CTA's row groups in shared memory and written as one fp32 partial row per
// CTA; a second kernel adds the partial rows in a fixed order.  That replaces
// the reference's spin-lock accumulation (rmsnorm_cached.py:245-264) by a
// deterministic two-stage reduce.
#include <mutex>

#include "common.cuh"

namespace rgd {

enum RowOp { L2_FWD = 0, L2_BWD = 1, RMS_FWD = 2, RMS_BWD = 3 };

constexpr int ROW_THREADS = 256;

struct RowStream {
    const void *x;
    const void *dy;
    void *out;        // y (forward) or dx (backward)
    const void *w;    // RMS only
    float *dw_part;   // RMS backward: [B][P][C] fp32 partial rows
    int64_t sxb, sxn, sdb, sdn, sob, son, swb;
    int N, C, P;      // rows per batch, channels, CTAs per batch
};

struct RowParams {
    RowStream s[2];
    int split;        // number of CTAs that belong to stream 0
    int tpr;          // threads per row (power of two, <= 256)
    int w_dtype;
    float eps;
};

// Sum over the `tpr` threads of a row group.  `red` is 2 x 8 floats of shared
// memory used alternately (`phase` toggles) when a group spans several warps.
__device__ __forceinline__ float group_sum(float v, int tpr, float (*red)[8], int &phase) {
    v = warp_group_sum(v, tpr < 32 ? tpr : 32);
    if (tpr > 32) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        if (lane == 0) red[phase][warp] = v;
        __syncthreads();
        const int wpg = tpr >> 5;
        const int first = (warp / wpg) * wpg;
        float t = 0.f;
        for (int i = 0; i < wpg; ++i) t += red[phase][first + i];
        v = t;
        phase ^= 1;
    }
    return v;
}

// T: element type.  VE: elements per access (16 bytes / sizeof(T), or 1 for
// rows that are not 16-byte addressable).  VPT: column slots per thread.
// PIPE: the 16-byte pieces of the next ROW_STAGES-1 rows are kept in flight with
// cp.async into per-thread shared-memory slots while the current row is
// processed (each thread reads back only slots it filled itself).
constexpr int ROW_STAGES = 3;

__device__ __forceinline__ void row_cp_async16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(gsrc)
                 : "memory");
}

template <typename T, int VE, int VPT, int OP, bool PIPE>
__global__ void __launch_bounds__(ROW_THREADS) row_kernel(const __grid_constant__ RowParams p) {
    constexpr bool BWD = (OP == L2_BWD || OP == RMS_BWD);
    constexpr bool RMS = (OP == RMS_FWD || OP == RMS_BWD);
    constexpr int SLOTS = (BWD ? 2 : 1) * VPT;
    using V = Vec<T, VE>;
    extern __shared__ uint4 row_slots[];                 // PIPE: [ROW_STAGES][SLOTS][ROW_THREADS]

    __shared__ float red[2][8];
    __shared__ float dwred[OP == RMS_BWD ? ROW_THREADS * VE : 1];
    int phase = 0;

    const int sid = (int)blockIdx.x >= p.split ? 1 : 0;
    const RowStream &s = p.s[sid];
    const int local = (int)blockIdx.x - (sid ? p.split : 0);
    const int b = local / s.P;
    const int chunk = local - b * s.P;
    const int tpr = p.tpr;
    const int rpc = ROW_THREADS / tpr;
    const int rg = (int)threadIdx.x / tpr;
    const int t = (int)threadIdx.x - rg * tpr;
    const int C = s.C;
    const float invC = 1.0f / (float)C;

    float wv[RMS ? VPT * VE : 1];
    float dwacc[OP == RMS_BWD ? VPT * VE : 1];
    if (RMS) {
#pragma unroll
        for (int j = 0; j < VPT; ++j)
#pragma unroll
            for (int e = 0; e < VE; ++e) {
                const int col = (t + j * tpr) * VE + e;
                wv[j * VE + e] = col < C ? load_as_f32(s.w, (int64_t)b * s.swb + col, p.w_dtype) : 0.f;
            }
    }
    if (OP == RMS_BWD) {
#pragma unroll
        for (int i = 0; i < VPT * VE; ++i) dwacc[i] = 0.f;
    }

    const T *xb = reinterpret_cast<const T *>(s.x) + (int64_t)b * s.sxb;
    const T *db = BWD ? reinterpret_cast<const T *>(s.dy) + (int64_t)b * s.sdb : nullptr;
    T *ob = reinterpret_cast<T *>(s.out) + (int64_t)b * s.sob;

    const int step = s.P * rpc;
    const int iters = (s.N + step - 1) / step;
    auto slot = [&](int stage, int idx) -> uint4 * {
        return row_slots + ((size_t)stage * SLOTS + idx) * ROW_THREADS + threadIdx.x;
    };
    auto issue = [&](int it, int stage) {
        const int n = it * step + chunk * rpc + rg;
        if (n >= s.N) return;
        const T *xr = xb + (int64_t)n * s.sxn;
        const T *dr = BWD ? db + (int64_t)n * s.sdn : nullptr;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int col = (t + j * tpr) * VE;
            if (col < C) {
                row_cp_async16(slot(stage, j), xr + col);
                if (BWD) row_cp_async16(slot(stage, VPT + j), dr + col);
            }
        }
    };
    if constexpr (PIPE) {
#pragma unroll
        for (int st = 0; st < ROW_STAGES - 1; ++st) {
            if (st < iters) issue(st, st);
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    }
    int stage = 0;
    for (int it = 0; it < iters; ++it) {
        const int n = it * step + chunk * rpc + rg;
        const bool valid = n < s.N;
        const T *xr = xb + (int64_t)n * s.sxn;
        const T *dr = BWD ? db + (int64_t)n * s.sdn : nullptr;

        V xq[VPT];
        V dq[BWD ? VPT : 1];
        if constexpr (PIPE) {
            int fill = stage + ROW_STAGES - 1;
            if (fill >= ROW_STAGES) fill -= ROW_STAGES;
            if (it + ROW_STAGES - 1 < iters) issue(it + ROW_STAGES - 1, fill);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group %0;" ::"n"(ROW_STAGES - 1) : "memory");
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int col = (t + j * tpr) * VE;
            if (valid && col < C) {
                if constexpr (PIPE) {
                    union { uint4 u; V v; } cx;
                    cx.u = *slot(stage, j);
                    xq[j] = cx.v;
                    if (BWD) {
                        cx.u = *slot(stage, VPT + j);
                        dq[j] = cx.v;
                    }
                } else {
                    xq[j] = load_vec<T, VE>(xr + col);
                    if (BWD) dq[j] = load_vec<T, VE>(dr + col);
                }
            } else {
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    xq[j].v[e] = from_f32<T>(0.f);
                    if (BWD) dq[j].v[e] = from_f32<T>(0.f);
                }
            }
        }
        if constexpr (PIPE) {
            if (++stage == ROW_STAGES) stage = 0;
        }

        // fp32 copies, converted once
        constexpr int NE = VPT * VE;
        float xf[NE];
        float df[BWD ? NE : 1];
#pragma unroll
        for (int j = 0; j < VPT; ++j)
#pragma unroll
            for (int e = 0; e < VE; ++e) {
                xf[j * VE + e] = to_f32<T>(xq[j].v[e]);
                if (BWD) df[j * VE + e] = to_f32<T>(dq[j].v[e]);
            }

        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < NE; ++i) ss = fmaf(xf[i], xf[i], ss);
        ss = group_sum(ss, tpr, red, phase);

        // Row scale: rmsnorm_cached.py:75-76, l2normalize_cached.py:72-77.
        float r;
        if (RMS) {
            r = rsqrtf(ss * invC + p.eps);
        } else {
            const float len = sqrtf(ss);
            r = (len < p.eps) ? (1.0f / p.eps) : (1.0f / len);
        }

        T *orow = ob + (int64_t)n * s.son;
        if (!BWD) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int col = (t + j * tpr) * VE;
                V yo;
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    float v = xf[j * VE + e] * r;
                    if (RMS) v = v * wv[j * VE + e];
                    yo.v[e] = from_f32<T>(v);
                }
                if (valid && col < C) store_vec_stream<T, VE>(orow + col, yo);
            }
        } else {
            // xhat, then g = sum(xhat * dy * w) [/ C for RMS]: rmsnorm_cached.py:213-231,
            // l2normalize_cached.py:214-226.
            float g = 0.f;
#pragma unroll
            for (int i = 0; i < NE; ++i) {
                xf[i] *= r;
                g += RMS ? xf[i] * df[i] * wv[i] : xf[i] * df[i];
            }
            g = group_sum(g, tpr, red, phase);
            if (RMS) g *= invC;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int col = (t + j * tpr) * VE;
                V yo;
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    const int i = j * VE + e;
                    float v;
                    if (RMS) {
                        v = (df[i] * wv[i] - xf[i] * g) * r;
                        if (OP == RMS_BWD) dwacc[i] += xf[i] * df[i];   // zero for padded rows
                    } else {
                        v = (df[i] - xf[i] * g) * r;
                    }
                    yo.v[e] = from_f32<T>(v);
                }
                if (valid && col < C) store_vec_stream<T, VE>(orow + col, yo);
            }
        }
    }

    if (OP == RMS_BWD) {
        // Fold the CTA's row groups together, one column slot at a time, and
        // write this CTA's partial row.
        float *prow = s.dw_part + ((int64_t)b * s.P + chunk) * C;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            __syncthreads();
#pragma unroll
            for (int e = 0; e < VE; ++e) dwred[threadIdx.x * VE + e] = dwacc[j * VE + e];
            __syncthreads();
            if (rg == 0) {
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    float a = 0.f;
                    for (int g2 = 0; g2 < rpc; ++g2) a += dwred[(g2 * tpr + t) * VE + e];
                    const int col = (t + j * tpr) * VE + e;
                    if (col < C) prow[col] = a;
                }
            }
        }
    }
}

// A 16-byte vector of the weight as fp32, whatever the weight's dtype.
template <typename T, int VE>
__device__ __forceinline__ void load_w_vec(const void *w, int64_t idx, int w_dtype, float (&out)[VE]) {
    if (w_dtype == DTypeCode<T>::value) {
        const Vec<T, VE> v = load_vec<T, VE>(reinterpret_cast<const T *>(w) + idx);
#pragma unroll
        for (int e = 0; e < VE; ++e) out[e] = to_f32<T>(v.v[e]);
    } else if (w_dtype == RGD_F32) {
        const float4 *src = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(w) + idx);
#pragma unroll
        for (int q = 0; q < VE / 4; ++q) {
            const float4 f = __ldg(src + q);
            out[4 * q] = f.x; out[4 * q + 1] = f.y; out[4 * q + 2] = f.z; out[4 * q + 3] = f.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < VE; ++e) out[e] = load_as_f32(w, idx + e, w_dtype);
    }
}

// ---------------------------------------------------------------------------
// Lean kernel for rows of exactly 128 * VPT vectors (four warps per row, two rows per CTA
// and iteration).  The pipelined kernel above spends about three quarters of its issue
// slots on bookkeeping (column and row predicates, 64-bit address arithmetic per vector,
// copy-pipeline slots), and at these row lengths issue slots are what bounds it.  Here the
// shape is exact, so there are no predicates; addresses advance by one add per row; the next
// row's vectors are loaded into registers before the current row is processed; and the two
// row groups of a CTA synchronise separately (named barriers), so neither waits for the other.
// Same CTA -> (tensor, batch, chunk) mapping, arithmetic and evaluation order as row_kernel.
// ---------------------------------------------------------------------------
constexpr int LEAN_TPR = 128;   // narrow form: 128 threads per row, two rows per CTA

// Makes the compiler forget what it derived from a 16-byte register vector, so that a later
// pass converts the raw elements again instead of keeping fp32 copies of the whole row alive.
template <typename V>
__device__ __forceinline__ void forget_derived(V &v) {
    static_assert(sizeof(V) == 16, "16-byte vectors only");
    uint4 &u = reinterpret_cast<uint4 &>(v);
    asm volatile("" : "+r"(u.x), "+r"(u.y), "+r"(u.z), "+r"(u.w));
}

template <int ID, int THREADS>
__device__ __forceinline__ void named_bar_sync() {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "n"(THREADS) : "memory");
}

// TPR threads per row, RPC rows per CTA and iteration (CTA = TPR * RPC threads), VPT vectors per
// thread.
template <typename T, int VPT, int OP, int TPR, int RPC>
// (three CTAs per SM for the forward operators: more rows in flight per SM; the backward ones,
// which hold x and dy of two rows, stay at two)
__global__ void __launch_bounds__(TPR * RPC, (OP == RMS_BWD || OP == L2_BWD) ? 2 : 3) lean_row_kernel(const __grid_constant__ RowParams p) {
    constexpr int THREADS = TPR * RPC;
    constexpr bool BWD = (OP == L2_BWD || OP == RMS_BWD);
    constexpr bool RMS = (OP == RMS_FWD || OP == RMS_BWD);
    constexpr int VE = VecElems<T>::value;
    constexpr int WPR = TPR / 32;                     // warps per row
    constexpr int NE = VPT * VE;
    using V = Vec<T, VE>;
    __shared__ float red[2][THREADS / 32];
    __shared__ float dwred[(OP == RMS_BWD && RPC > 1) ? THREADS * VE : 1];
    // RMS backward: the fp32 weight row sits in shared memory ([VPT][TPR][VE]) and is read
    // per use, which with the raw-register passes below keeps the kernel at 2 CTAs per SM.
    __shared__ __align__(16) float wsm[OP == RMS_BWD ? TPR * NE : 1];

    const int sid = (int)blockIdx.x >= p.split ? 1 : 0;
    const RowStream &s = p.s[sid];
    const int local = (int)blockIdx.x - (sid ? p.split : 0);
    const int b = local / s.P;
    const int chunk = local - b * s.P;
    const int warp = (int)threadIdx.x >> 5, lane = (int)threadIdx.x & 31;
    const int rg = (int)threadIdx.x / TPR;
    const int t = (int)threadIdx.x - rg * TPR;
    const float invC = 1.0f / (float)s.C;
    int phase = 0;

    auto group_sum = [&](float v) -> float {
        v = warp_group_sum(v, 32);
        if (lane == 0) red[phase][warp] = v;
        if (rg == 0) named_bar_sync<1, TPR>();             // literal ids: the compiler reserves only these
        else named_bar_sync<2, TPR>();
        float a = 0.f;
#pragma unroll
        for (int i = 0; i < WPR; ++i) a += red[phase][rg * WPR + i];
        phase ^= 1;
        return a;
    };

    float wv[OP == RMS_FWD ? NE : 1];
    float dwacc[OP == RMS_BWD ? NE : 1];
    if (RMS) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            float w8[VE];
            load_w_vec<T, VE>(s.w, (int64_t)b * s.swb + (t + j * TPR) * VE, p.w_dtype, w8);
#pragma unroll
            for (int e = 0; e < VE; ++e) {
                if (OP == RMS_FWD) wv[j * VE + e] = w8[e];
                else if (rg == 0) wsm[(j * TPR + t) * VE + e] = w8[e];
            }
        }
    }
    if (OP == RMS_BWD) {
#pragma unroll
        for (int i = 0; i < NE; ++i) dwacc[i] = 0.f;
        __syncthreads();
    }
    auto w_slot = [&](int j, float (&w8)[VE]) {            // this thread's weights of vector j
        const float4 *src = reinterpret_cast<const float4 *>(wsm + (j * TPR + t) * VE);
#pragma unroll
        for (int q = 0; q < VE / 4; ++q) {
            const float4 f = src[q];
            w8[4 * q] = f.x; w8[4 * q + 1] = f.y; w8[4 * q + 2] = f.z; w8[4 * q + 3] = f.w;
        }
    };

    const int step = s.P * RPC;
    int n = chunk * RPC + rg;
    const T *xr = reinterpret_cast<const T *>(s.x) + (int64_t)b * s.sxb + (int64_t)n * s.sxn + t * VE;
    const T *dr = BWD ? reinterpret_cast<const T *>(s.dy) + (int64_t)b * s.sdb + (int64_t)n * s.sdn + t * VE : nullptr;
    T *orow = reinterpret_cast<T *>(s.out) + (int64_t)b * s.sob + (int64_t)n * s.son + t * VE;
    const int64_t xstep = (int64_t)step * s.sxn, dstep = BWD ? (int64_t)step * s.sdn : 0, ostep = (int64_t)step * s.son;

    // The next row of this group is in flight while the current one is processed.  (Measured
    // for the RMS backward on B200 at configuration 5 and not kept: two rows ahead, by register
    // copies or by rotating buffers through an unrolled loop, 60-73 us against 42 us; weight
    // row AND dweight sums in shared memory, 53 us.  Kept: weight row in shared memory plus
    // raw-register passes, two CTAs per SM, 40 us.)
    // The dweight reduce that follows the RMS backward is launched as a programmatic dependent:
    // let it be set up now; it waits for this grid's completion before it reads anything.
    if constexpr (OP == RMS_BWD) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    V xq[VPT], xn[VPT];
    V dq[BWD ? VPT : 1], dn[BWD ? VPT : 1];
    if (n < s.N) {
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            xq[j] = load_vec_stream<T, VE>(xr + j * TPR * VE);
            if (BWD) dq[j] = load_vec_stream<T, VE>(dr + j * TPR * VE);
        }
    }
    for (; n < s.N; n += step) {
        if (n + step < s.N) {
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                xn[j] = load_vec_stream<T, VE>(xr + xstep + j * TPR * VE);
                if (BWD) dn[j] = load_vec_stream<T, VE>(dr + dstep + j * TPR * VE);
            }
        }
        if constexpr (OP == RMS_BWD) {
            // Three passes over the raw 16-bit (or fp32) registers, converting again in each:
            // fp32 copies of x and dy kept across the two row sums would cost 2 * NE registers
            // and with them the second CTA per SM.  Same arithmetic and order as below.
            float ss = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j)
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    const float xf = to_f32<T>(xq[j].v[e]);
                    ss = fmaf(xf, xf, ss);
                }
            ss = group_sum(ss);
#pragma unroll
            for (int j = 0; j < VPT; ++j) forget_derived(xq[j]);
            const float r = rsqrtf(ss * invC + p.eps);
            float g = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                float w8[VE];
                w_slot(j, w8);
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    const float xh = to_f32<T>(xq[j].v[e]) * r;
                    g += xh * to_f32<T>(dq[j].v[e]) * w8[e];
                }
            }
            g = group_sum(g) * invC;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                forget_derived(xq[j]);
                forget_derived(dq[j]);
            }
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                V yo;
                float w8[VE];
                w_slot(j, w8);
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    const int i = j * VE + e;
                    const float xh = to_f32<T>(xq[j].v[e]) * r;
                    const float df = to_f32<T>(dq[j].v[e]);
                    yo.v[e] = from_f32<T>((df * w8[e] - xh * g) * r);
                    dwacc[i] += xh * df;
                }
                store_vec_stream<T, VE>(orow + j * TPR * VE, yo);
            }
        } else {
            float xf[NE];
            float df[BWD ? NE : 1];
    #pragma unroll
            for (int j = 0; j < VPT; ++j)
    #pragma unroll
                for (int e = 0; e < VE; ++e) {
                    xf[j * VE + e] = to_f32<T>(xq[j].v[e]);
                    if (BWD) df[j * VE + e] = to_f32<T>(dq[j].v[e]);
                }
            float ss = 0.f;
    #pragma unroll
            for (int i = 0; i < NE; ++i) ss = fmaf(xf[i], xf[i], ss);
            ss = group_sum(ss);

            // Row scale: rmsnorm_cached.py:75-76, l2normalize_cached.py:72-77.
            float r;
            if (RMS) {
                r = rsqrtf(ss * invC + p.eps);
            } else {
                const float len = sqrtf(ss);
                r = (len < p.eps) ? (1.0f / p.eps) : (1.0f / len);
            }

            if (!BWD) {
    #pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    V yo;
    #pragma unroll
                    for (int e = 0; e < VE; ++e) {
                        float y = xf[j * VE + e] * r;
                        if (RMS) y = y * wv[j * VE + e];
                        yo.v[e] = from_f32<T>(y);
                    }
                    store_vec_stream<T, VE>(orow + j * TPR * VE, yo);
                }
            } else {
                // xhat, then g = sum(xhat * dy * w) [/ C for RMS]: rmsnorm_cached.py:213-231,
                // l2normalize_cached.py:214-226.
                float g = 0.f;
    #pragma unroll
                for (int i = 0; i < NE; ++i) {
                    xf[i] *= r;
                    g += xf[i] * df[i];                         // (the RMS backward took the branch above)
                }
                g = group_sum(g);
                if (RMS) g *= invC;
    #pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    V yo;
    #pragma unroll
                    for (int e = 0; e < VE; ++e) {
                        const int i = j * VE + e;
                        float dxv;
                        dxv = (df[i] - xf[i] * g) * r;
                        yo.v[e] = from_f32<T>(dxv);
                    }
                    store_vec_stream<T, VE>(orow + j * TPR * VE, yo);
                }
            }
        }
        xr += xstep;
        if (BWD) dr += dstep;
        orow += ostep;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            xq[j] = xn[j];
            if (BWD) dq[j] = dn[j];
        }
    }

    if (OP == RMS_BWD) {
        // Fold the CTA's row groups together, one column slot at a time, and write this CTA's
        // partial row.
        float *prow = s.dw_part + ((int64_t)b * s.P + chunk) * s.C;
        if (RPC == 1) {
#pragma unroll
            for (int j = 0; j < VPT; ++j)
#pragma unroll
                for (int e = 0; e < VE; ++e) prow[(t + j * TPR) * VE + e] = dwacc[j * VE + e];
            return;
        }
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            __syncthreads();
#pragma unroll
            for (int e = 0; e < VE; ++e) dwred[threadIdx.x * VE + e] = dwacc[j * VE + e];
            __syncthreads();
            if (rg == 0) {
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    float a = 0.f;
#pragma unroll
                    for (int g2 = 0; g2 < RPC; ++g2) a += dwred[(g2 * TPR + t) * VE + e];
                    prow[(t + j * TPR) * VE + e] = a;
                }
            }
        }
    }
}

// Geometry of the lean kernel for rows of `nvec` vectors: 128 threads per row, 2..4 vectors per
// thread, two rows per CTA.  (A wide form, one vector per thread and the whole CTA on one row,
// was measured for the RMS backward: 65 instead of 171 registers, but the same bytes in flight
// per SM and the same 42-44 us at configuration 5, so it is not kept.)
struct LeanGeom {
    bool ok;
    int tpr, rpc, vpt;
};
template <int OP>
LeanGeom lean_geometry(int nvec) {
    if (nvec % LEAN_TPR == 0 && nvec / LEAN_TPR >= 2 && nvec / LEAN_TPR <= 4) return {true, LEAN_TPR, 2, nvec / LEAN_TPR};
    return {false, 0, 0, 0};
}

// F(kernel, threads) for the instantiation that matches the geometry.
template <typename T, int OP, typename F>
int with_lean_kernel(const LeanGeom &g, F f) {
    if (g.rpc != 2 || g.tpr != LEAN_TPR) return RGD_E_SIZE;
    switch (g.vpt) {
        case 2: return f(lean_row_kernel<T, 2, OP, LEAN_TPR, 2>, 2 * LEAN_TPR);
        case 3: return f(lean_row_kernel<T, 3, OP, LEAN_TPR, 2>, 2 * LEAN_TPR);
        case 4: return f(lean_row_kernel<T, 4, OP, LEAN_TPR, 2>, 2 * LEAN_TPR);
    }
    return RGD_E_SIZE;
}

template <typename T, int OP>
int launch_lean_rows(const RowParams &p, const LeanGeom &g, int grid, cudaStream_t st) {
    return with_lean_kernel<T, OP>(g, [&](auto kernel, int threads) {
        kernel<<<grid, threads, 0, st>>>(p);
        count_launch();
        return check_launch();
    });
}

template <int OP>
int launch_lean_rows_dtype(int dtype, const RowParams &p, const LeanGeom &g, int grid, cudaStream_t st) {
    switch (dtype) {
        case RGD_F32: return launch_lean_rows<float, OP>(p, g, grid, st);
        case RGD_F16: return launch_lean_rows<__half, OP>(p, g, grid, st);
        case RGD_BF16: return launch_lean_rows<__nv_bfloat16, OP>(p, g, grid, st);
    }
    return RGD_E_DTYPE;
}

// CTAs of the lean kernel resident on one SM.
template <typename T, int OP>
int lean_rows_occupancy_t(const LeanGeom &g) {
    int n = 0;
    const int rc = with_lean_kernel<T, OP>(g, [&](auto kernel, int threads) {
        n = cached_occupancy(reinterpret_cast<const void *>(kernel), threads, 0);
        return 0;
    });
    if (rc != 0 || n < 1) n = 1;
    return n;
}
template <int OP>
int lean_rows_occupancy(int dtype, const LeanGeom &g) {
    switch (dtype) {
        case RGD_F32: return lean_rows_occupancy_t<float, OP>(g);
        case RGD_F16: return lean_rows_occupancy_t<__half, OP>(g);
    }
    return lean_rows_occupancy_t<__nv_bfloat16, OP>(g);
}

// Second stage of dweight: dw[b or -, c] = sum over partial rows, fixed order.
// blockDim = (32 columns, 32 row lanes); grid = (ceil(C/32), B or 1, streams).
struct DwReduceStream {
    const float *part;   // [rows_total][C]
    void *dw;            // [B or 1][C] in w dtype
    int C;
    int rows_per_out;    // partial rows folded into one output row
    int n_out;           // output rows (B for per-batch weights, else 1)
};
struct DwReduceParams {
    DwReduceStream s[2];
    int w_dtype;
};

__global__ void __launch_bounds__(1024) dw_reduce_kernel(const __grid_constant__ DwReduceParams p) {
    __shared__ float tile[32][33];
    // Launched as a programmatic dependent of the kernel that writes the partial rows: the grid may
    // be set up while that kernel drains; nothing is read before it has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const DwReduceStream &s = p.s[blockIdx.z];
    const int o = blockIdx.y;
    if (o >= s.n_out) return;
    const int col = blockIdx.x * 32 + threadIdx.x;
    if (blockIdx.x * 32 >= s.C) return;
    float a = 0.f;
    if (col < s.C) {
        const float *base = s.part + (int64_t)o * s.rows_per_out * s.C + col;
        // four independent loads in flight per thread (a fixed order all the same): with one
        // the kernel is a chain of L2 round trips
        float a1 = 0.f, a2 = 0.f, a3 = 0.f;
        int r = threadIdx.y;
        for (; r + 96 < s.rows_per_out; r += 128) {
            a += base[(int64_t)r * s.C];
            a1 += base[(int64_t)(r + 32) * s.C];
            a2 += base[(int64_t)(r + 64) * s.C];
            a3 += base[(int64_t)(r + 96) * s.C];
        }
        for (; r < s.rows_per_out; r += 32) a += base[(int64_t)r * s.C];
        a = (a + a1) + (a2 + a3);
    }
    tile[threadIdx.y][threadIdx.x] = a;
    __syncthreads();
    if (threadIdx.y == 0 && col < s.C) {
        float t = 0.f;
#pragma unroll
        for (int r = 0; r < 32; ++r) t += tile[r][threadIdx.x];
        store_from_f32(s.dw, (int64_t)o * s.C + col, p.w_dtype, t);
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace {

struct RowPlan {
    int ve;    // 1 or 16/sizeof(T)
    int vpt;   // template slot count
    int tpr;
};

// Pick the access width, threads per row and slots per thread for rows of
// `cmax` channels.  Returns false when the row does not fit in registers.
bool plan_rows(int cmax, int esize, bool vector_ok, RowPlan &pl) {
    const int ve = vector_ok ? 16 / esize : 1;
    const int nvec = (cmax + ve - 1) / ve;
    int tpr = next_pow2(nvec);
    if (tpr > 32) tpr = 32;
    int vpt = (nvec + tpr - 1) / tpr;
    while (vpt > 4 && tpr < ROW_THREADS) {
        tpr <<= 1;
        vpt = (nvec + tpr - 1) / tpr;
    }
    const int vmax = vector_ok ? 8 : 32;
    if (vpt > vmax) return false;
    if (vector_ok) {
        if (vpt > 4) vpt = 8;
    } else {
        vpt = vpt <= 4 ? 4 : 32;
    }
    pl.ve = ve;
    pl.vpt = vpt;
    pl.tpr = tpr;
    return true;
}

// Shared memory of the pipelined kernel for VPT slots per thread.
template <int OP>
constexpr size_t row_pipe_smem(int vpt) {
    return (size_t)ROW_STAGES * ((OP == L2_BWD || OP == RMS_BWD) ? 2 : 1) * vpt * ROW_THREADS * 16;
}

template <typename T, int VE, int VPT, int OP, bool PIPE>
int launch_row_kernel(const RowParams &p, int grid, cudaStream_t st) {
    auto kernel = row_kernel<T, VE, VPT, OP, PIPE>;
    const size_t smem = PIPE ? row_pipe_smem<OP>(VPT) : 0;
    if (smem > 32 * 1024)   // static shared memory counts towards the 48 KB default limit too
        if (int e = ensure_dyn_smem(reinterpret_cast<const void *>(kernel), smem)) return e;
    kernel<<<grid, ROW_THREADS, smem, st>>>(p);
    count_launch();
    return check_launch();
}

// CTAs of this instantiation that are resident on one SM at the same time.
template <typename T, int VE, int VPT, int OP, bool PIPE>
int row_kernel_occupancy() {
    auto kernel = row_kernel<T, VE, VPT, OP, PIPE>;
    const size_t smem = PIPE ? row_pipe_smem<OP>(VPT) : 0;
    if (smem > 32 * 1024)
        (void)ensure_dyn_smem(reinterpret_cast<const void *>(kernel), smem);
    return cached_occupancy(reinterpret_cast<const void *>(kernel), ROW_THREADS, smem);
}

template <typename T, int OP>
int rows_occupancy(const RowPlan &pl) {
    constexpr int VE = VecElems<T>::value;
    if (pl.ve == 1) return 0;
    switch (pl.vpt) {
        case 1: return row_kernel_occupancy<T, VE, 1, OP, true>();
        case 2: return row_kernel_occupancy<T, VE, 2, OP, true>();
        case 3: return row_kernel_occupancy<T, VE, 3, OP, true>();
        case 4: return row_kernel_occupancy<T, VE, 4, OP, true>();
    }
    return 0;
}

template <int OP>
int rows_occupancy_dtype(int dtype, const RowPlan &pl) {
    switch (dtype) {
        case RGD_F32: return rows_occupancy<float, OP>(pl);
        case RGD_F16: return rows_occupancy<__half, OP>(pl);
        case RGD_BF16: return rows_occupancy<__nv_bfloat16, OP>(pl);
    }
    return 0;
}

template <typename T, int VE, int OP>
int launch_rows_vpt(const RowParams &p, int vpt, int grid, cudaStream_t st) {
    switch (vpt) {
        case 1: return launch_row_kernel<T, VE, 1, OP, true>(p, grid, st);
        case 2: return launch_row_kernel<T, VE, 2, OP, true>(p, grid, st);
        case 3: return launch_row_kernel<T, VE, 3, OP, true>(p, grid, st);
        case 4: return launch_row_kernel<T, VE, 4, OP, true>(p, grid, st);
        case 8: return launch_row_kernel<T, VE, 8, OP, false>(p, grid, st);
    }
    return RGD_E_SIZE;
}

template <typename T, int OP>
int launch_rows_scalar(const RowParams &p, int vpt, int grid, cudaStream_t st) {
    if (vpt == 4) return launch_row_kernel<T, 1, 4, OP, false>(p, grid, st);
    if (vpt == 32) return launch_row_kernel<T, 1, 32, OP, false>(p, grid, st);
    return RGD_E_SIZE;
}

template <typename T, int OP>
int launch_rows(const RowParams &p, const RowPlan &pl, int grid, cudaStream_t st) {
    if (pl.ve == 1) return launch_rows_scalar<T, OP>(p, pl.vpt, grid, st);
    return launch_rows_vpt<T, VecElems<T>::value, OP>(p, pl.vpt, grid, st);
}

template <int OP>
int launch_rows_dtype(int dtype, const RowParams &p, const RowPlan &pl, int grid, cudaStream_t st) {
    switch (dtype) {
        case RGD_F32: return launch_rows<float, OP>(p, pl, grid, st);
        case RGD_F16: return launch_rows<__half, OP>(p, pl, grid, st);
        case RGD_BF16: return launch_rows<__nv_bfloat16, OP>(p, pl, grid, st);
    }
    return RGD_E_DTYPE;
}

bool view_vec_ok(const rgd_rows &v, int esize) {
    const int ve = 16 / esize;
    return is_aligned(v.ptr, 16) && v.stride_b % ve == 0 && v.stride_n % ve == 0;
}

// CTAs per batch for each stream.  `budget` is the total CTA count aimed at.
void split_ctas(int nstreams, const int64_t *N, int64_t B, int rpc, int budget, int *P) {
    int64_t groups[2] = {0, 0}, total = 0;
    for (int s = 0; s < nstreams; ++s) {
        groups[s] = ceil_div64(N[s], rpc);
        total += groups[s] * B;
    }
    for (int s = 0; s < nstreams; ++s) {
        int64_t ps = groups[s];
        if (total > budget) {
            // proportional share per batch, rounded DOWN so the whole grid stays within
            // the budget (one resident wave; a few CTAs over it would cost a second wave)
            ps = groups[s] * budget / total;
            if (ps < 1) ps = 1;
            if (ps > groups[s]) ps = groups[s];
        }
        if (ps < 1) ps = 1;
        // Even out the walk: with k = ceil(groups / ps) iterations per CTA, ceil(groups / k)
        // CTAs do the same work in the same k iterations and none of them idles through a
        // mostly empty last iteration (2048 row groups over 444 CTAs: 5 iterations at 92%;
        // over 410 CTAs: 5 iterations at 99.9%).
        if (groups[s] > 0) {
            const int64_t k = ceil_div64(groups[s], ps);
            ps = ceil_div64(groups[s], k);
        }
        P[s] = (int)ps;
    }
}

struct RowCall {
    int nstreams;
    const rgd_rows *x, *dy, *out;
    const void *const *w;
    const int64_t *wsb;
    const int64_t *N, *C;
    int64_t B;
    float eps;
    int x_dtype, w_dtype;
};

int validate_rows(const RowCall &c, bool bwd, bool rms) {
    if (c.nstreams < 1 || c.nstreams > 2) return RGD_E_INVALID;
    if (!c.x || !c.out || !c.N || !c.C) return RGD_E_NULL;
    if (bwd && !c.dy) return RGD_E_NULL;
    if (rms && (!c.w || !c.wsb)) return RGD_E_NULL;
    if (!dtype_ok(c.x_dtype)) return RGD_E_DTYPE;
    if (rms && !dtype_ok(c.w_dtype)) return RGD_E_DTYPE;
    if (c.B < 0 || c.B > INT32_MAX) return RGD_E_INVALID;
    for (int s = 0; s < c.nstreams; ++s) {
        if (c.N[s] < 0 || c.C[s] < 0 || c.N[s] > INT32_MAX || c.C[s] > INT32_MAX) return RGD_E_INVALID;
        const bool empty = c.B == 0 || c.N[s] == 0 || c.C[s] == 0;
        if (!empty) {
            if (!c.x[s].ptr || !c.out[s].ptr) return RGD_E_NULL;
            if (bwd && !c.dy[s].ptr) return RGD_E_NULL;
        }
        if (rms && c.C[s] > 0 && !c.w[s]) return RGD_E_NULL;
    }
    return RGD_OK;
}

// Build the launch for one of the four row operators.  *plan_out / *P_out
// return the chosen geometry (needed by the dweight reduce).
template <int OP>
int run_rows(const RowCall &c, float *dw_part0, float *dw_part1, int budget, cudaStream_t st, int *P_out) {
    constexpr bool BWD = (OP == L2_BWD || OP == RMS_BWD);
    const int esize = dtype_size(c.x_dtype);
    int cmax = 0;
    bool vec_ok = true;
    for (int s = 0; s < c.nstreams; ++s) {
        if (c.C[s] > cmax) cmax = (int)c.C[s];
        vec_ok = vec_ok && (c.C[s] % (16 / esize) == 0) && view_vec_ok(c.x[s], esize) && view_vec_ok(c.out[s], esize);
        if (BWD) vec_ok = vec_ok && view_vec_ok(c.dy[s], esize);
    }
    RowPlan pl;
    if (!plan_rows(cmax > 0 ? cmax : 1, esize, vec_ok, pl)) return RGD_E_SIZE;

    RowParams p{};
    p.tpr = pl.tpr;
    p.w_dtype = c.w_dtype;
    p.eps = c.eps;
    int P[2] = {0, 0};
    const int nvec = pl.ve > 1 ? (cmax + pl.ve - 1) / pl.ve : 0;
    // Rows of exactly 128 * {2, 3, 4} vectors in every tensor: the lean kernel.
    const LeanGeom lg = lean_geometry<OP>(nvec);
    bool lean_rows = pl.ve > 1 && lg.ok && cmax % pl.ve == 0;
    for (int s = 0; s < c.nstreams; ++s) lean_rows = lean_rows && (c.C[s] == cmax || c.N[s] == 0);
    // The lean kernel reads the weight with 16-byte loads: its address and batch stride
    // must allow that; any other weight view takes the pipelined kernel (scalar weight loads).
    if (c.w) {
        const int wvec = 16 / dtype_size(c.w_dtype);
        for (int s = 0; s < c.nstreams; ++s)
            lean_rows = lean_rows && (c.N[s] == 0 || (is_aligned(c.w[s], 16) && c.wsb[s] % wvec == 0));
    }
    int rows_per_cta = ROW_THREADS / pl.tpr;
    if (lean_rows) {
        pl.tpr = lg.tpr;
        rows_per_cta = lg.rpc;
        const int resident = lean_rows_occupancy<OP>(c.x_dtype, lg) * num_sms();
        if (OP != RMS_BWD || resident < budget) budget = resident;
    } else if (pl.ve > 1 && pl.vpt <= 4) {
        // Pipelined kernel: launch exactly one resident wave, so every CTA streams
        // several rows and the copy pipeline stays full.
        const int per_sm = rows_occupancy_dtype<OP>(c.x_dtype, pl);
        if (per_sm > 0) {
            const int resident = per_sm * num_sms();
            if (OP != RMS_BWD || resident < budget) budget = resident;
        }
    }
    if (!lean_rows) rows_per_cta = ROW_THREADS / pl.tpr;
    split_ctas(c.nstreams, c.N, c.B, rows_per_cta, budget, P);
    int64_t grid = 0;
    for (int s = 0; s < c.nstreams; ++s) {
        RowStream &rs = p.s[s];
        rs.x = c.x[s].ptr;
        rs.sxb = c.x[s].stride_b;
        rs.sxn = c.x[s].stride_n;
        rs.out = c.out[s].ptr;
        rs.sob = c.out[s].stride_b;
        rs.son = c.out[s].stride_n;
        if (BWD) {
            rs.dy = c.dy[s].ptr;
            rs.sdb = c.dy[s].stride_b;
            rs.sdn = c.dy[s].stride_n;
        }
        if (c.w) {
            rs.w = c.w[s];
            rs.swb = c.wsb[s];
        }
        rs.dw_part = s == 0 ? dw_part0 : dw_part1;
        rs.N = (int)c.N[s];
        rs.C = (int)c.C[s];
        // A stream with no rows or no channels gets no CTAs.
        const bool empty = c.N[s] == 0 || c.C[s] == 0;
        rs.P = empty ? 0 : P[s];
        if (rs.P == 0) rs.P = 1, P[s] = 0; else P[s] = rs.P;
        const int64_t ctas = (int64_t)P[s] * c.B;
        if (s == 0) p.split = (int)ctas;
        grid += ctas;
    }
    if (P_out) { P_out[0] = P[0]; P_out[1] = P[1]; }
    if (grid == 0) return RGD_OK;
    if (grid > INT32_MAX) return RGD_E_SIZE;
    if (lean_rows) return launch_lean_rows_dtype<OP>(c.x_dtype, p, lg, (int)grid, st);
    return launch_rows_dtype<OP>(c.x_dtype, p, pl, (int)grid, st);
}

constexpr int FWD_CTAS_PER_SM = 16;
constexpr int BWD_CTAS_PER_SM = 4;

}  // namespace

}  // namespace rgd

using namespace rgd;

extern "C" int rgd_l2norm_fwd(int nstreams, const rgd_rows *x, const rgd_rows *y, const int64_t *N,
                              const int64_t *C, int64_t B, float eps, int dtype, void *stream) {
    RowCall c{nstreams, x, nullptr, y, nullptr, nullptr, N, C, B, eps, dtype, RGD_F32};
    if (int e = validate_rows(c, false, false)) return e;
    return run_rows<L2_FWD>(c, nullptr, nullptr, FWD_CTAS_PER_SM * num_sms(), (cudaStream_t)stream, nullptr);
}

extern "C" int rgd_l2norm_bwd(int nstreams, const rgd_rows *x, const rgd_rows *dy, const rgd_rows *dx,
                              const int64_t *N, const int64_t *C, int64_t B, float eps, int dtype,
                              void *stream) {
    RowCall c{nstreams, x, dy, dx, nullptr, nullptr, N, C, B, eps, dtype, RGD_F32};
    if (int e = validate_rows(c, true, false)) return e;
    return run_rows<L2_BWD>(c, nullptr, nullptr, FWD_CTAS_PER_SM * num_sms(), (cudaStream_t)stream, nullptr);
}

extern "C" int rgd_rmsnorm_fwd(int nstreams, const rgd_rows *x, const void *const *w,
                               const int64_t *w_stride_b, const rgd_rows *y, const int64_t *N,
                               const int64_t *C, int64_t B, float eps, int x_dtype, int w_dtype,
                               void *stream) {
    RowCall c{nstreams, x, nullptr, y, w, w_stride_b, N, C, B, eps, x_dtype, w_dtype};
    if (int e = validate_rows(c, false, true)) return e;
    return run_rows<RMS_FWD>(c, nullptr, nullptr, FWD_CTAS_PER_SM * num_sms(), (cudaStream_t)stream, nullptr);
}

// Upper bound of partial rows per stream: never more CTAs than the budget.
static int64_t rms_bwd_part_rows() { return (int64_t)BWD_CTAS_PER_SM * num_sms(); }

extern "C" int64_t rgd_rmsnorm_bwd_workspace_bytes(int nstreams, const int64_t *N, const int64_t *C,
                                                   int64_t B) {
    if (nstreams < 1 || nstreams > 2 || !N || !C || B < 0) return RGD_E_INVALID;
    int64_t bytes = 0;
    for (int s = 0; s < nstreams; ++s) {
        // P[s] * B <= budget + B (each stream keeps at least one CTA per batch).
        const int64_t rows = rms_bwd_part_rows() + B;
        bytes += rows * C[s] * (int64_t)sizeof(float);
        bytes = (bytes + 255) / 256 * 256;
    }
    return bytes;
}

extern "C" int rgd_rmsnorm_bwd(int nstreams, const rgd_rows *x, const void *const *w,
                               const int64_t *w_stride_b, const rgd_rows *dy, const rgd_rows *dx,
                               void *const *dw, const int *dw_per_batch, const int64_t *N,
                               const int64_t *C, int64_t B, float eps, int x_dtype, int w_dtype,
                               void *workspace, int64_t workspace_bytes, void *stream) {
    RowCall c{nstreams, x, dy, dx, w, w_stride_b, N, C, B, eps, x_dtype, w_dtype};
    if (int e = validate_rows(c, true, true)) return e;
    if (!dw || !dw_per_batch) return RGD_E_NULL;
    const int64_t need = rgd_rmsnorm_bwd_workspace_bytes(nstreams, N, C, B);
    if (need > 0 && (!workspace || workspace_bytes < need)) return RGD_E_WORKSPACE;
    if (need > 0 && !is_aligned(workspace, 16)) return RGD_E_STRIDE;

    float *part[2] = {nullptr, nullptr};
    {
        int64_t off = 0;
        for (int s = 0; s < nstreams; ++s) {
            part[s] = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + off);
            off += (rms_bwd_part_rows() + B) * C[s] * (int64_t)sizeof(float);
            off = (off + 255) / 256 * 256;
        }
    }
    int P[2] = {0, 0};
    cudaStream_t st = (cudaStream_t)stream;
    if (int e = run_rows<RMS_BWD>(c, part[0], part[1], (int)rms_bwd_part_rows(), st, P)) return e;

    // Second stage.  A stream without rows still has to produce dw = 0.
    DwReduceParams rp{};
    rp.w_dtype = w_dtype;
    int cmax = 0, omax = 0;
    for (int s = 0; s < nstreams; ++s) {
        if (C[s] > 0 && !dw[s]) return RGD_E_NULL;
        DwReduceStream &d = rp.s[s];
        d.part = part[s];
        d.dw = dw[s];
        d.C = (int)C[s];
        if (dw_per_batch[s]) {
            d.n_out = (int)B;
            d.rows_per_out = P[s];
        } else {
            d.n_out = B > 0 ? 1 : 0;
            d.rows_per_out = P[s] * (int)B;
        }
        if (d.C > cmax) cmax = d.C;
        if (d.n_out > omax) omax = d.n_out;
    }
    if (cmax == 0 || omax == 0) return RGD_OK;
    dim3 grid((cmax + 31) / 32, omax, nstreams), block(32, 32);
    {
        // programmatic dependent launch: the reduce grid is set up while the row kernel drains
        // (it waits for that kernel's completion before reading); a plain launch if refused
        cudaLaunchConfig_t cfg{};
        cfg.gridDim = grid;
        cfg.blockDim = block;
        cfg.dynamicSmemBytes = 0;
        cfg.stream = st;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cudaLaunchKernelEx(&cfg, dw_reduce_kernel, rp) != cudaSuccess) {
            (void)cudaGetLastError();
            dw_reduce_kernel<<<grid, block, 0, st>>>(rp);
        }
    }
    count_launch();
    return check_launch();
}

// ---------------------------------------------------------------------------
// RMSNorm backward without any allocation by anybody.
//
// rgd_rmsnorm_bwd needs a scratch buffer for its per-CTA dweight partial rows,
// which the caller normally allocates.  Some callers cannot allocate device
// memory at the point where they need the backward: a plugin inside a host
// application that hands out all device memory at start-up and forbids
// cudaMalloc afterwards, or a section of a serving / training loop that must
// not incur the implicit device synchronisation and latency of an allocation.
// For them the scratch lives in this fixed-size device array, which every GPU
// that loads the library holds from load until the process exits.
//
// The array's name is usable directly only in device code.  On the host it is a
// stand-in, not a device address, so the address is fetched once per device
// with cudaGetSymbolAddress (with that device current) and passed on.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_rms_bwd_static_scratch[RGD_RMSNORM_BWD_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mutex;
void *g_static_scratch_addr[64] = {nullptr};

// Device address of the static scratch on the CURRENT device; looked up on the
// first call per device, cached afterwards.  Returns a status code.
int static_scratch_address(void **out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_status(e);
    if (dev < 0 || dev >= 64) return RGD_E_DEVICE;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_addr[dev] == nullptr) {
        void *ptr = nullptr;
        e = cudaGetSymbolAddress((void **)&ptr, g_rms_bwd_static_scratch);
        if (e != cudaSuccess) {
            (void)cudaGetLastError();
            return cuda_status(e);
        }
        g_static_scratch_addr[dev] = ptr;
    }
    *out = g_static_scratch_addr[dev];
    return RGD_OK;
}
}  // namespace

extern "C" int rgd_rmsnorm_bwd_static(int nstreams, const rgd_rows *x, const void *const *w,
                                      const int64_t *w_stride_b, const rgd_rows *dy, const rgd_rows *dx,
                                      void *const *dw, const int *dw_per_batch, const int64_t *N,
                                      const int64_t *C, int64_t B, float eps, int x_dtype, int w_dtype,
                                      void *stream) {
    // Same argument checks, in the same order, as the workspace form: a bad size or a null
    // pointer is reported as such before anything is sized or looked up.
    RowCall c{nstreams, x, dy, dx, w, w_stride_b, N, C, B, eps, x_dtype, w_dtype};
    if (int e = validate_rows(c, true, true)) return e;
    if (!dw || !dw_per_batch) return RGD_E_NULL;
    const int64_t need = rgd_rmsnorm_bwd_workspace_bytes(nstreams, N, C, B);
    if (need < 0) return RGD_E_INVALID;
    // Sizes whose partial rows do not fit the fixed array are refused, not truncated.
    if (need > (int64_t)RGD_RMSNORM_BWD_STATIC_SCRATCH_BYTES) return RGD_E_WORKSPACE;
    void *scratch = nullptr;
    if (int e = static_scratch_address(&scratch)) return e;
    // Nothing in the scratch has to start at zero: every partial row the reduce
    // reads is first written in full by the CTA that owns it.
    return rgd_rmsnorm_bwd(nstreams, x, w, w_stride_b, dy, dx, dw, dw_per_batch, N, C, B, eps, x_dtype, w_dtype,
                           scratch, (int64_t)RGD_RMSNORM_BWD_STATIC_SCRATCH_BYTES, stream);
}
