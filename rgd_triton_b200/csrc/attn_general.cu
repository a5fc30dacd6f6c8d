// General FlashAttention kernels (forward, delta, dK/dV, dQ) on mma.sync
// tensor-core instructions.  They take every shape the operator accepts:
// head_dim 1..128 (zero-padded to 32 / 64 / 128 in shared memory), any
// sequence lengths, arbitrary element strides with a contiguous channel axis,
// vector or matrix bias in the tensor dtype or fp32 with stride-0 broadcast
// dims, causal masking.  The tensor-memory kernels take over for the aligned
// head_dim 64 / 128 cases; this file is the path for everything else.
//
// Numerics follow flash_attn_triton_cached.py: S = QK^T accumulated in fp32,
// S*scale + bias, online softmax in fp32, P and dS rounded to the tensor
// dtype before their second GEMM (:208, :492, :510), fp32 accumulators, one
// rounding on store.  The backward is split into a dK/dV kernel (one CTA per
// key block) and a dQ kernel (one CTA per query block), so every output
// element is produced by exactly one CTA in a fixed order: no atomics, results
// are bit-reproducible from run to run.
#include <math.h>

#include "attn_mma.cuh"

namespace rgd {
namespace attn {

template <typename T, int DPAD>
struct alignas(16) FwdSmem {
    Tile<T, DPAD> q, k, v;
};
template <typename T, int DPAD>
struct alignas(16) BwdSmem {
    Tile<T, DPAD> q, k, v, d_o;
    float lse[64];
    float delta[64];
};

__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// ---------------------------------------------------------------------------
// Forward: one CTA per (64 query rows, batch*head).
// ---------------------------------------------------------------------------
template <typename T, int DPAD>
__global__ void __launch_bounds__(NTHREADS) attn_fwd_general(const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FwdSmem<T, DPAD> &sm = *reinterpret_cast<FwdSmem<T, DPAD> *>(smem_raw);

    const int mblk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m0 = mblk * BM;
    const int rows_valid = min(BM, p.Tq - m0);

    const T *qp = reinterpret_cast<const T *>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)m0 * p.q_sn;
    const T *kp = reinterpret_cast<const T *>(p.k) + (int64_t)b * p.k_sb + (int64_t)h * p.k_sh;
    const T *vp = reinterpret_cast<const T *>(p.v) + (int64_t)b * p.v_sb + (int64_t)h * p.v_sh;
    const char *bias_bh = nullptr;
    if (p.bias_kind != RGD_BIAS_NONE)
        bias_bh = reinterpret_cast<const char *>(p.bias) +
                  ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : (int)sizeof(T));

    load_tile<T, DPAD>(sm.q, qp, p.q_sn, rows_valid, p.d, p.vec_q);

    float acc[DPAD / 8][4];
#pragma unroll
    for (int i = 0; i < DPAD / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    float mrow[2] = {-INFINITY, -INFINITY}, lrow[2] = {0.f, 0.f};
    const int row[2] = {m0 + warp * 16 + g, m0 + warp * 16 + g + 8};

    const int n_end = p.causal ? min(p.Tk, m0 + BM) : p.Tk;
    for (int n0 = 0; n0 < n_end; n0 += BN) {
        __syncthreads();
        const int kv_valid = min(BN, p.Tk - n0);
        load_tile<T, DPAD>(sm.k, kp + (int64_t)n0 * p.k_sn, p.k_sn, kv_valid, p.d, p.vec_k);
        load_tile<T, DPAD>(sm.v, vp + (int64_t)n0 * p.v_sn, p.v_sn, kv_valid, p.d, p.vec_v);
        __syncthreads();

        float s[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = 0.f;
        gemm_nt<T, DPAD>(s, sm.q, warp * 16, sm.k);

        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int col = n0 + nt * 8 + 2 * t + (e & 1);
                const int r = row[e >> 1];
                float v = s[nt][e] * p.scale;
                if (bias_bh != nullptr && r < p.Tq && col < p.Tk) v += bias_at_t<T>(p, bias_bh, r, col);
                if (col >= p.Tk || (p.causal && col > r)) v = -INFINITY;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], muse[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const float mnew = fmaxf(mrow[hh], quad_max(mx[hh]));
            muse[hh] = (mnew == -INFINITY) ? 0.f : mnew;
            alpha[hh] = exp2f((mrow[hh] - muse[hh]) * LOG2E);
            mrow[hh] = mnew;
        }
        float ls[2] = {0.f, 0.f};
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float pv = exp2f((s[nt][e] - muse[e >> 1]) * LOG2E);
                s[nt][e] = pv;
                ls[e >> 1] += pv;
            }
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) lrow[hh] = lrow[hh] * alpha[hh] + ls[hh];
#pragma unroll
        for (int i = 0; i < DPAD / 8; ++i) {
            acc[i][0] *= alpha[0];
            acc[i][1] *= alpha[0];
            acc[i][2] *= alpha[1];
            acc[i][3] *= alpha[1];
        }
        uint32_t pf[4][4];
        pack_p<T>(pf, s);
        gemm_pn<T, DPAD>(acc, pf, sm.v);
    }

    float inv[2], lse[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const float l = quad_sum(lrow[hh]);
        inv[hh] = l > 0.f ? 1.0f / l : 0.f;
        lse[hh] = l > 0.f ? mrow[hh] + logf(l) : -INFINITY;
    }
    T *op = reinterpret_cast<T *>(p.out_o) + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh +
            (int64_t)(m0 + warp * 16) * p.o_sn;
    store_acc<T, DPAD>(acc, op, p.o_sn, rows_valid - warp * 16, p.d, p.vec_o, inv[0], inv[1]);
    if (t == 0) {
        float *lp = p.lse + (int64_t)bh * p.Tq_rounded;
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
            if (row[hh] < p.Tq_rounded) lp[row[hh]] = row[hh] < p.Tq ? lse[hh] : INFINITY;
    }
}

// ---------------------------------------------------------------------------
// delta[b,h,i] = sum_c O[i,c] * dO[i,c]   (flash_attn_triton_cached.py:249-292)
// One warp per row; rows in [Tq, Tq_rounded) get 0.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) attn_delta_kernel(const __grid_constant__ AttnParams p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i = blockIdx.x * 8 + warp;
    const int bh = blockIdx.y;
    if (i >= p.Tq_rounded) return;
    const int b = bh / p.H, h = bh - b * p.H;
    float a = 0.f;
    if (i < p.Tq) {
        const T *o = reinterpret_cast<const T *>(p.o) + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)i * p.o_sn;
        const T *g = reinterpret_cast<const T *>(p.d_o) + (int64_t)b * p.do_sb + (int64_t)h * p.do_sh +
                     (int64_t)i * p.do_sn;
        for (int c = lane; c < p.d; c += 32) a += to_f32<T>(o[c]) * to_f32<T>(g[c]);
    }
    a = warp_group_sum(a, 32);
    if (lane == 0) p.delta[(int64_t)bh * p.Tq_rounded + i] = a;
}

// ---------------------------------------------------------------------------
// dK, dV: one CTA per (64 keys, batch*head), loop over query blocks.  The tile
// is kept transposed (keys x queries) so that P^T and dS^T come out of the
// tensor cores already laid out as the A operand of the dV / dK GEMMs.
// ---------------------------------------------------------------------------
template <typename T, int DPAD>
__global__ void __launch_bounds__(NTHREADS) attn_bwd_kv_general(const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BwdSmem<T, DPAD> &sm = *reinterpret_cast<BwdSmem<T, DPAD> *>(smem_raw);

    const int nblk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = nblk * BN;
    const int kv_valid = min(BN, p.Tk - n0);

    const T *qp = reinterpret_cast<const T *>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh;
    const T *gp = reinterpret_cast<const T *>(p.d_o) + (int64_t)b * p.do_sb + (int64_t)h * p.do_sh;
    const T *kp = reinterpret_cast<const T *>(p.k) + (int64_t)b * p.k_sb + (int64_t)h * p.k_sh + (int64_t)n0 * p.k_sn;
    const T *vp = reinterpret_cast<const T *>(p.v) + (int64_t)b * p.v_sb + (int64_t)h * p.v_sh + (int64_t)n0 * p.v_sn;
    const float *lse = p.lse + (int64_t)bh * p.Tq_rounded;
    const float *delta = p.delta + (int64_t)bh * p.Tq_rounded;
    const char *bias_bh = nullptr;
    if (p.bias_kind != RGD_BIAS_NONE)
        bias_bh = reinterpret_cast<const char *>(p.bias) +
                  ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : (int)sizeof(T));

    load_tile<T, DPAD>(sm.k, kp, p.k_sn, kv_valid, p.d, p.vec_k);
    load_tile<T, DPAD>(sm.v, vp, p.v_sn, kv_valid, p.d, p.vec_v);

    float acc_dv[DPAD / 8][4], acc_dk[DPAD / 8][4];
#pragma unroll
    for (int i = 0; i < DPAD / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_dv[i][e] = acc_dk[i][e] = 0.f;
    const int krow[2] = {n0 + warp * 16 + g, n0 + warp * 16 + g + 8};
    float dbs[2] = {0.f, 0.f};   // vector-bias gradient: sum over the queries of P (dP - delta) per key row

    // Causal: queries before this key block see none of its keys.
    const int m_begin = p.causal ? (n0 / BM) * BM : 0;
    for (int m0 = m_begin; m0 < p.Tq; m0 += BM) {
        __syncthreads();
        const int q_valid = min(BM, p.Tq - m0);
        load_tile<T, DPAD>(sm.q, qp + (int64_t)m0 * p.q_sn, p.q_sn, q_valid, p.d, p.vec_q);
        load_tile<T, DPAD>(sm.d_o, gp + (int64_t)m0 * p.do_sn, p.do_sn, q_valid, p.d, p.vec_do);
        if (threadIdx.x < 64) {
            const int i = m0 + threadIdx.x;
            sm.lse[threadIdx.x] = i < p.Tq ? lse[i] : INFINITY;
            sm.delta[threadIdx.x] = i < p.Tq ? delta[i] : 0.f;
        }
        __syncthreads();

        float st[8][4], dpt[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) st[i][e] = dpt[i][e] = 0.f;
        gemm_nt<T, DPAD>(st, sm.k, warp * 16, sm.q);      // S^T  = K Q^T
        gemm_nt<T, DPAD>(dpt, sm.v, warp * 16, sm.d_o);   // dP^T = V dO^T

#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int ql = nt * 8 + 2 * t + (e & 1);
                const int qi = m0 + ql;
                const int kj = krow[e >> 1];
                float v = st[nt][e] * p.scale;
                const bool masked = kj >= p.Tk || qi >= p.Tq || (p.causal && kj > qi);
                if (bias_bh != nullptr && !masked) v += bias_at_t<T>(p, bias_bh, qi, kj);
                const float pv = masked ? 0.f : exp2f((v - sm.lse[ql]) * LOG2E);
                st[nt][e] = pv;                                            // P^T
                const float dsr = pv * (dpt[nt][e] - sm.delta[ql]);
                dbs[e >> 1] += dsr;
                dpt[nt][e] = dsr * p.scale;                                // dS^T
            }
        uint32_t pf[4][4];
        pack_p<T>(pf, st);
        gemm_pn<T, DPAD>(acc_dv, pf, sm.d_o);             // dV += P^T dO
        pack_p<T>(pf, dpt);
        gemm_pn<T, DPAD>(acc_dk, pf, sm.q);               // dK += dS^T Q
    }

    if (p.dbias != nullptr && p.bias_kind == RGD_BIAS_VECTOR) {
        // the four lanes of a quad hold the same two key rows; one add per key in the whole grid
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            float v = dbs[hh];
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            if (t == 0 && krow[hh] < p.Tk)
                atomicAdd(reinterpret_cast<float *>(p.dbias) + (int64_t)b * p.db_sb + (int64_t)h * p.db_sh + krow[hh], v);
        }
    }
    T *dvp = reinterpret_cast<T *>(p.dv) + (int64_t)b * p.dv_sb + (int64_t)h * p.dv_sh +
             (int64_t)(n0 + warp * 16) * p.dv_sn;
    T *dkp = reinterpret_cast<T *>(p.dk) + (int64_t)b * p.dk_sb + (int64_t)h * p.dk_sh +
             (int64_t)(n0 + warp * 16) * p.dk_sn;
    store_acc<T, DPAD>(acc_dv, dvp, p.dv_sn, kv_valid - warp * 16, p.d, p.vec_dv, 1.f, 1.f);
    store_acc<T, DPAD>(acc_dk, dkp, p.dk_sn, kv_valid - warp * 16, p.d, p.vec_dk, 1.f, 1.f);
}

// ---------------------------------------------------------------------------
// dQ: one CTA per (64 queries, batch*head), loop over key blocks.
// ---------------------------------------------------------------------------
template <typename T, int DPAD>
__global__ void __launch_bounds__(NTHREADS) attn_bwd_q_general(const __grid_constant__ AttnParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BwdSmem<T, DPAD> &sm = *reinterpret_cast<BwdSmem<T, DPAD> *>(smem_raw);

    const int mblk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m0 = mblk * BM;
    const int q_valid = min(BM, p.Tq - m0);

    const T *qp = reinterpret_cast<const T *>(p.q) + (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)m0 * p.q_sn;
    const T *gp = reinterpret_cast<const T *>(p.d_o) + (int64_t)b * p.do_sb + (int64_t)h * p.do_sh +
                  (int64_t)m0 * p.do_sn;
    const T *kp = reinterpret_cast<const T *>(p.k) + (int64_t)b * p.k_sb + (int64_t)h * p.k_sh;
    const T *vp = reinterpret_cast<const T *>(p.v) + (int64_t)b * p.v_sb + (int64_t)h * p.v_sh;
    const char *bias_bh = nullptr;
    if (p.bias_kind != RGD_BIAS_NONE)
        bias_bh = reinterpret_cast<const char *>(p.bias) +
                  ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : (int)sizeof(T));

    T *dbias_bh = nullptr;       // matrix-bias gradient: P (dP - delta) element by element
    if (p.dbias != nullptr && p.bias_kind == RGD_BIAS_MATRIX)
        dbias_bh = reinterpret_cast<T *>(p.dbias) + (int64_t)b * p.db_sb + (int64_t)h * p.db_sh;

    load_tile<T, DPAD>(sm.q, qp, p.q_sn, q_valid, p.d, p.vec_q);
    load_tile<T, DPAD>(sm.d_o, gp, p.do_sn, q_valid, p.d, p.vec_do);

    const int row[2] = {m0 + warp * 16 + g, m0 + warp * 16 + g + 8};
    float lse_r[2], delta_r[2];
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const bool ok = row[hh] < p.Tq;
        lse_r[hh] = ok ? p.lse[(int64_t)bh * p.Tq_rounded + row[hh]] : INFINITY;
        delta_r[hh] = ok ? p.delta[(int64_t)bh * p.Tq_rounded + row[hh]] : 0.f;
    }

    float acc[DPAD / 8][4];
#pragma unroll
    for (int i = 0; i < DPAD / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;

    const int n_end = p.causal ? min(p.Tk, m0 + BM) : p.Tk;
    for (int n0 = 0; n0 < n_end; n0 += BN) {
        __syncthreads();
        const int kv_valid = min(BN, p.Tk - n0);
        load_tile<T, DPAD>(sm.k, kp + (int64_t)n0 * p.k_sn, p.k_sn, kv_valid, p.d, p.vec_k);
        load_tile<T, DPAD>(sm.v, vp + (int64_t)n0 * p.v_sn, p.v_sn, kv_valid, p.d, p.vec_v);
        __syncthreads();

        float s[8][4], dp[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[i][e] = dp[i][e] = 0.f;
        gemm_nt<T, DPAD>(s, sm.q, warp * 16, sm.k);        // S  = Q K^T
        gemm_nt<T, DPAD>(dp, sm.d_o, warp * 16, sm.v);     // dP = dO V^T
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int kj = n0 + nt * 8 + 2 * t + (e & 1);
                const int qi = row[e >> 1];
                float v = s[nt][e] * p.scale;
                const bool masked = kj >= p.Tk || qi >= p.Tq || (p.causal && kj > qi);
                if (bias_bh != nullptr && !masked) v += bias_at_t<T>(p, bias_bh, qi, kj);
                const float pv = masked ? 0.f : exp2f((v - lse_r[e >> 1]) * LOG2E);
                const float dsr = pv * (dp[nt][e] - delta_r[e >> 1]);
                if (dbias_bh != nullptr && qi < p.Tq && kj < p.Tk) dbias_bh[(int64_t)qi * p.db_sq + kj] = from_f32<T>(dsr);
                s[nt][e] = dsr * p.scale;                                  // dS
            }
        uint32_t pf[4][4];
        pack_p<T>(pf, s);
        gemm_pn<T, DPAD>(acc, pf, sm.k);                   // dQ += dS K
    }
    T *dqp = reinterpret_cast<T *>(p.dq) + (int64_t)b * p.dq_sb + (int64_t)h * p.dq_sh +
             (int64_t)(m0 + warp * 16) * p.dq_sn;
    store_acc<T, DPAD>(acc, dqp, p.dq_sn, q_valid - warp * 16, p.d, p.vec_dq, 1.f, 1.f);
}

// ---------------------------------------------------------------------------
// Host dispatch
// ---------------------------------------------------------------------------
template <typename K>
static int set_smem(K kernel, size_t bytes) {
    if (bytes > 48 * 1024)
        return ensure_dyn_smem(reinterpret_cast<const void *>(kernel), bytes);
    return RGD_OK;
}

template <typename T, int DPAD>
static int fwd_launch(const AttnParams &p, cudaStream_t st) {
    const size_t smem = sizeof(FwdSmem<T, DPAD>);
    if (int e = set_smem(attn_fwd_general<T, DPAD>, smem)) return e;
    dim3 grid((p.Tq + BM - 1) / BM, p.B * p.H);
    attn_fwd_general<T, DPAD><<<grid, NTHREADS, smem, st>>>(p);
    count_launch();
    return check_launch();
}

template <typename T, int DPAD>
static int bwd_launch(const AttnParams &p, cudaStream_t st) {
    const size_t smem = sizeof(BwdSmem<T, DPAD>);
    if (int e = set_smem(attn_bwd_kv_general<T, DPAD>, smem)) return e;
    if (int e = set_smem(attn_bwd_q_general<T, DPAD>, smem)) return e;
    if (p.Tk > 0) {
        dim3 grid((p.Tk + BN - 1) / BN, p.B * p.H);
        attn_bwd_kv_general<T, DPAD><<<grid, NTHREADS, smem, st>>>(p);
        count_launch();
        if (int e = check_launch()) return e;
    }
    if (p.Tq > 0) {
        dim3 grid((p.Tq + BM - 1) / BM, p.B * p.H);
        attn_bwd_q_general<T, DPAD><<<grid, NTHREADS, smem, st>>>(p);
        count_launch();
        if (int e = check_launch()) return e;
    }
    return RGD_OK;
}

template <typename T>
static int fwd_dispatch(const AttnParams &p, cudaStream_t st) {
    if (p.d <= 32) return fwd_launch<T, 32>(p, st);
    if (p.d <= 64) return fwd_launch<T, 64>(p, st);
    return fwd_launch<T, 128>(p, st);
}

template <typename T>
static int bwd_dispatch(const AttnParams &p, cudaStream_t st) {
    if (p.Tq_rounded > 0) {
        dim3 grid((p.Tq_rounded + 7) / 8, p.B * p.H);
        attn_delta_kernel<T><<<grid, 256, 0, st>>>(p);
        count_launch();
        if (int e = check_launch()) return e;
    }
    if (p.d <= 32) return bwd_launch<T, 32>(p, st);
    if (p.d <= 64) return bwd_launch<T, 64>(p, st);
    return bwd_launch<T, 128>(p, st);
}

int general_fwd(const AttnParams &p, int dtype, cudaStream_t st) {
    if (p.B == 0 || p.H == 0 || p.Tq == 0) return RGD_OK;
    return dtype == RGD_F16 ? fwd_dispatch<__half>(p, st) : fwd_dispatch<__nv_bfloat16>(p, st);
}

int general_bwd(const AttnParams &p, int dtype, cudaStream_t st) {
    if (p.B == 0 || p.H == 0) return RGD_OK;
    return dtype == RGD_F16 ? bwd_dispatch<__half>(p, st) : bwd_dispatch<__nv_bfloat16>(p, st);
}

}  // namespace attn
}  // namespace rgd
