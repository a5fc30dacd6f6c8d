// Per-head row operators on Q and K in one launch: LayerNorm over head_dim
// (no affine), interleaved-pair rotary embedding on the first R channels of
// the first `cut` tokens, and the fused LayerNorm -> rotary, each forward and
// backward.
//
// A row is the head_dim channels of one (batch, head, token).  Rows are walked
// in MEMORY order (the dimension with the smaller stride innermost), so with a
// [B, N, H, d] tensor the H*d channels of a token are read as one contiguous
// run and with [B, H, N, d] the N*d run of a head is — either way every warp
// access is fully coalesced.  `tpr` consecutive threads own one row with one
// 16-byte access each; each thread handles ROWS_PER_THREAD independent rows so
// several loads are in flight before the first reduction.  Row statistics are
// recomputed in the backward pass from x (which the backward reads anyway), so
// no statistics buffer exists.
#include "common.cuh"

namespace rgd {

enum HeadOp { LN_FWD = 0, LN_BWD = 1, ROPE = 2, LNROPE_FWD = 3, LNROPE_BWD = 4 };

constexpr int HEAD_THREADS = 256;
constexpr int ROWS_PER_THREAD = 4;

struct HeadTensor {
    const void *x;
    const void *dy;
    void *out;
    // element strides for (batch, outer, inner) of x, dy, out
    int64_t xb, x1, x2, db, d1, d2, ob, o1, o2;
    int D1, D2;         // extents of the outer / inner row dimension
    int seq_inner;      // 1 when the inner dimension is the token axis
    int cut;            // tokens that get the rotation
    int64_t rows;       // B * D1 * D2
};

struct HeadParams {
    HeadTensor t[2];
    int64_t split;      // CTAs that belong to tensor 0
    int d;              // head_dim
    int tpr;            // threads per row (power of two <= 32)
    int R;              // rotary channels
    const void *pos;    // [2, P, R]: sin, cos
    int64_t pos_ss, pos_sn;
    int transposed;     // rotary: apply the inverse rotation
    float eps;
};

// Load VE table entries starting at column `col` (col < R guaranteed for the
// first entry; entries at or beyond R read as 0).
template <typename TP, int VE>
__device__ __forceinline__ void load_table(const TP *row, int col, int R, bool vec_ok, float *out) {
    if (VE > 1 && vec_ok && col + VE <= R) {
        constexpr int PER = 16 / sizeof(TP);            // table elements per 16-byte access
        constexpr int NACC = (VE + PER - 1) / PER;
        constexpr int W = VE < PER ? VE : PER;
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
            Vec<TP, W> v = load_vec<TP, W>(row + col + a * W);
#pragma unroll
            for (int e = 0; e < W; ++e) out[a * W + e] = to_f32<TP>(v.v[e]);
        }
    } else {
#pragma unroll
        for (int e = 0; e < VE; ++e) out[e] = (col + e < R) ? to_f32<TP>(row[col + e]) : 0.f;
    }
}

// T: tensor element type.  TP: table element type (T or float).  VE: elements
// per access (16 / sizeof(T), or 1).  VPT: column slots per thread.
template <typename T, typename TP, int VE, int VPT, int OP>
__global__ void __launch_bounds__(HEAD_THREADS, (OP == LN_BWD || OP == LNROPE_BWD) ? 3 : 4) head_kernel(const __grid_constant__ HeadParams p) {
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    constexpr bool HAS_ROPE = (OP == ROPE || OP == LNROPE_FWD || OP == LNROPE_BWD);
    constexpr bool HAS_LN = (OP != ROPE);
    // The stand-alone rotary computes in the promoted type of x and the table
    // (head_rope_cached.py:48,142): 16-bit x with a 16-bit table rounds after
    // every multiply and add; anything else is plain fp32.
    constexpr bool ROUND_EACH = (OP == ROPE) && (sizeof(T) == 2) && (sizeof(TP) == 2);
    using V = Vec<T, VE>;
    constexpr int NE = VPT * VE;

    const int ti = (int64_t)blockIdx.x >= p.split ? 1 : 0;
    const HeadTensor &ht = p.t[ti];
    const int64_t local = (int64_t)blockIdx.x - (ti ? p.split : 0);
    const int tpr = p.tpr;
    const int rpc = HEAD_THREADS / tpr;                 // rows per CTA pass
    const int rg = (int)threadIdx.x / tpr;
    const int t = (int)threadIdx.x - rg * tpr;
    const int d = p.d;
    const float invd = 1.0f / (float)d;
    const bool pos_vec_ok = (reinterpret_cast<uintptr_t>(p.pos) % 16 == 0) &&
                            (p.pos_ss % (16 / (int)sizeof(TP)) == 0) && (p.pos_sn % (16 / (int)sizeof(TP)) == 0);

    // Loaded rows stay packed (16 bytes per slot) until their turn to be
    // processed: that keeps the register count low enough for 4 CTAs per SM.
    V xq[ROWS_PER_THREAD][VPT];
    V gq[HAS_DY ? ROWS_PER_THREAD : 1][VPT];
    int64_t ooff[ROWS_PER_THREAD];
    int tok[ROWS_PER_THREAD];
    bool valid[ROWS_PER_THREAD];

    // ---- issue all loads first --------------------------------------------
#pragma unroll
    for (int r = 0; r < ROWS_PER_THREAD; ++r) {
        const int64_t rid = (local * ROWS_PER_THREAD + r) * rpc + rg;
        valid[r] = rid < ht.rows;
        const int64_t rr = valid[r] ? rid : 0;
        int i1, i2;
        int64_t b;
        if (ht.rows <= 0x7fffffffLL) {             // 32-bit divisions for every realistic size
            const unsigned r32 = (unsigned)rr;
            const unsigned q1 = r32 / (unsigned)ht.D2;
            i2 = (int)(r32 - q1 * (unsigned)ht.D2);
            const unsigned q2 = q1 / (unsigned)ht.D1;
            i1 = (int)(q1 - q2 * (unsigned)ht.D1);
            b = q2;
        } else {
            i2 = (int)(rr % ht.D2);
            const int64_t q1 = rr / ht.D2;
            i1 = (int)(q1 % ht.D1);
            b = q1 / ht.D1;
        }
        tok[r] = ht.seq_inner ? i2 : i1;
        const T *xr = reinterpret_cast<const T *>(ht.x) + b * ht.xb + (int64_t)i1 * ht.x1 + (int64_t)i2 * ht.x2;
        const T *dr = HAS_DY ? reinterpret_cast<const T *>(ht.dy) + b * ht.db + (int64_t)i1 * ht.d1 + (int64_t)i2 * ht.d2
                             : nullptr;
        ooff[r] = b * ht.ob + (int64_t)i1 * ht.o1 + (int64_t)i2 * ht.o2;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int col = (t + j * tpr) * VE;
            if (valid[r] && col < d) {
                xq[r][j] = load_vec_stream<T, VE>(xr + col);
                if constexpr (HAS_DY) gq[r][j] = load_vec_stream<T, VE>(dr + col);
            } else {
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    xq[r][j].v[e] = from_f32<T>(0.f);
                    if constexpr (HAS_DY) gq[r][j].v[e] = from_f32<T>(0.f);
                }
            }
        }
    }

    // ---- per row -------------------------------------------------------------
#pragma unroll
    for (int r = 0; r < ROWS_PER_THREAD; ++r) {
        float xv[NE];
        float dv[HAS_DY ? NE : 1];
#pragma unroll
        for (int j = 0; j < VPT; ++j)
#pragma unroll
            for (int e = 0; e < VE; ++e) {
                xv[j * VE + e] = to_f32<T>(xq[r][j].v[e]);
                if constexpr (HAS_DY) dv[j * VE + e] = to_f32<T>(gq[r][j].v[e]);
            }
        float mean = 0.f, rstd = 1.f;
        if (HAS_LN) {
            // head_layernorm_cached.py:85-99 / fused_ln_rope_cached.py:66-74
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < NE; ++i) s += xv[i];
            mean = warp_group_sum(s, tpr) * invd;
            float s2 = 0.f;
#pragma unroll
            for (int j = 0; j < VPT; ++j)
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    const int col = (t + j * tpr) * VE + e;
                    const float c = col < d ? xv[j * VE + e] - mean : 0.f;
                    xv[j * VE + e] = c;           // centred
                    s2 += c * c;
                }
            rstd = rsqrtf(warp_group_sum(s2, tpr) * invd + p.eps);
#pragma unroll
            for (int i = 0; i < NE; ++i) xv[i] *= rstd;   // xhat
        }

        const bool rot_row = HAS_ROPE && tok[r] < ht.cut;
        float res[NE];

        // Scalar mode: the rotation partner (channel c ^ 1) lives in the
        // neighbouring lane.  Exchange it unconditionally so that every lane
        // of the warp takes part in the shuffle.
        float oth[(VE == 1 && HAS_ROPE) ? NE : 1];
        if constexpr (VE == 1 && HAS_ROPE) {
#pragma unroll
            for (int j = 0; j < NE; ++j) {
                float mine;
                if constexpr (OP == LNROPE_BWD) mine = dv[j]; else mine = xv[j];
                oth[j] = __shfl_xor_sync(0xffffffffu, mine, 1);
            }
        }

        if constexpr (OP == LN_FWD) {
#pragma unroll
            for (int i = 0; i < NE; ++i) res[i] = xv[i];
        } else if constexpr (OP == LN_BWD || OP == LNROPE_BWD) {
            float *g = dv;
            if constexpr (OP == LNROPE_BWD) {
                if (rot_row) {
                    // Inverse rotation of the upstream gradient (fused_ln_rope_cached.py:349-360).
                    const TP *srow = reinterpret_cast<const TP *>(p.pos) + (int64_t)tok[r] * p.pos_sn;
                    const TP *crow = srow + p.pos_ss;
#pragma unroll
                    for (int j = 0; j < VPT; ++j) {
                        const int col = (t + j * tpr) * VE;
                        if (col < p.R) {
                            float sn[VE], cs[VE];
                            load_table<TP, VE>(srow, col, p.R, pos_vec_ok, sn);
                            load_table<TP, VE>(crow, col, p.R, pos_vec_ok, cs);
                            if constexpr (VE > 1) {
#pragma unroll
                                for (int e = 0; e < VE; e += 2) {
                                    const float ge = g[j * VE + e], go = g[j * VE + e + 1];
                                    if (col + e < p.R) g[j * VE + e] = ge * cs[e] + go * sn[e];
                                    if (col + e + 1 < p.R) g[j * VE + e + 1] = go * cs[e + 1] - ge * sn[e + 1];
                                }
                            } else {
                                const float me = g[j];
                                g[j] = (col & 1) ? me * cs[0] - oth[j] * sn[0] : me * cs[0] + oth[j] * sn[0];
                            }
                        }
                    }
                }
            }
            // head_layernorm_cached.py:193-199 / fused_ln_rope_cached.py:100-114
            float sa = 0.f, sb = 0.f;
#pragma unroll
            for (int i = 0; i < NE; ++i) {
                sa += xv[i] * g[i];
                sb += g[i];
            }
            const float a = warp_group_sum(sa, tpr) * invd;
            const float bm = warp_group_sum(sb, tpr) * invd;
#pragma unroll
            for (int i = 0; i < NE; ++i) res[i] = (g[i] - xv[i] * a - bm) * rstd;
        } else {
            // ROPE or LNROPE_FWD: rotate xv (raw x, or xhat).
#pragma unroll
            for (int i = 0; i < NE; ++i) res[i] = xv[i];
            if (rot_row) {
                const TP *srow = reinterpret_cast<const TP *>(p.pos) + (int64_t)tok[r] * p.pos_sn;
                const TP *crow = srow + p.pos_ss;
                const bool inv = (OP == ROPE) && p.transposed;
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const int col = (t + j * tpr) * VE;
                    if (col < p.R) {
                        float sn[VE], cs[VE];
                        load_table<TP, VE>(srow, col, p.R, pos_vec_ok, sn);
                        load_table<TP, VE>(crow, col, p.R, pos_vec_ok, cs);
                        if constexpr (VE > 1) {
#pragma unroll
                            for (int e = 0; e < VE; e += 2) {
                                const float xe = xv[j * VE + e], xo = xv[j * VE + e + 1];
                                // rotated partner: (-x_odd, x_even), sign flipped for the inverse
                                const float re = inv ? xo : -xo;
                                const float ro = inv ? -xe : xe;
                                float oe, oo;
                                if constexpr (ROUND_EACH) {
                                    oe = round_to<T>(round_to<T>(xe * cs[e]) + round_to<T>(re * sn[e]));
                                    oo = round_to<T>(round_to<T>(xo * cs[e + 1]) + round_to<T>(ro * sn[e + 1]));
                                } else {
                                    oe = xe * cs[e] + re * sn[e];
                                    oo = xo * cs[e + 1] + ro * sn[e + 1];
                                }
                                if (col + e < p.R) res[j * VE + e] = oe;
                                if (col + e + 1 < p.R) res[j * VE + e + 1] = oo;
                            }
                        } else {
                            const float me = xv[j];
                            float rot = (col & 1) ? oth[j] : -oth[j];
                            if (inv) rot = -rot;
                            if constexpr (ROUND_EACH)
                                res[j] = round_to<T>(round_to<T>(me * cs[0]) + round_to<T>(rot * sn[0]));
                            else
                                res[j] = me * cs[0] + rot * sn[0];
                        }
                    }
                }
            }
        }

        if (valid[r]) {
            T *orow = reinterpret_cast<T *>(ht.out) + ooff[r];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int col = (t + j * tpr) * VE;
                if (col < d) {
                    V o;
#pragma unroll
                    for (int e = 0; e < VE; ++e) o.v[e] = from_f32<T>(res[j * VE + e]);
                    store_vec_stream<T, VE>(orow + col, o);
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
namespace {

struct HeadCall {
    const rgd_heads *x[2];     // q, k inputs
    const rgd_heads *dy[2];    // upstream gradients (backward) or null
    const rgd_heads *out[2];
    int64_t B, H, N[2], d;
    const void *pos;
    int64_t pos_ss, pos_sn, P, R, cut[2];
    int transposed;
    float eps;
    int x_dtype, pos_dtype;
};

bool heads_vec_ok(const rgd_heads &v, int esize) {
    const int ve = 16 / esize;
    return is_aligned(v.ptr, 16) && v.stride_b % ve == 0 && v.stride_h % ve == 0 && v.stride_n % ve == 0;
}

template <typename T, typename TP, int OP>
int launch_head(const HeadParams &p, bool vec, int vpt, int64_t grid, cudaStream_t st) {
    constexpr int VE = VecElems<T>::value;
    if (grid > INT32_MAX) return RGD_E_SIZE;
    if (vec) {
        if (vpt == 1)
            head_kernel<T, TP, VE, 1, OP><<<(unsigned)grid, HEAD_THREADS, 0, st>>>(p);
        else if (vpt == 2)
            head_kernel<T, TP, VE, 2, OP><<<(unsigned)grid, HEAD_THREADS, 0, st>>>(p);
        else
            return RGD_E_SIZE;
    } else {
        if (vpt <= 4)
            head_kernel<T, TP, 1, 4, OP><<<(unsigned)grid, HEAD_THREADS, 0, st>>>(p);
        else if (vpt <= 8)
            head_kernel<T, TP, 1, 8, OP><<<(unsigned)grid, HEAD_THREADS, 0, st>>>(p);
        else
            return RGD_E_SIZE;
    }
    count_launch();
    return check_launch();
}

template <int OP>
int dispatch_head(const HeadCall &c, const HeadParams &p, bool vec, int vpt, int64_t grid, cudaStream_t st) {
    constexpr bool USES_TABLE = (OP == ROPE || OP == LNROPE_FWD || OP == LNROPE_BWD);
    const bool tab32 = USES_TABLE && c.pos_dtype == RGD_F32;
    switch (c.x_dtype) {
        case RGD_F32:
            return launch_head<float, float, OP>(p, vec, vpt, grid, st);
        case RGD_F16:
            if (tab32) return launch_head<__half, float, OP>(p, vec, vpt, grid, st);
            return launch_head<__half, __half, OP>(p, vec, vpt, grid, st);
        case RGD_BF16:
            if (tab32) return launch_head<__nv_bfloat16, float, OP>(p, vec, vpt, grid, st);
            return launch_head<__nv_bfloat16, __nv_bfloat16, OP>(p, vec, vpt, grid, st);
    }
    return RGD_E_DTYPE;
}

template <int OP>
int run_head(const HeadCall &c, cudaStream_t st) {
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    constexpr bool USES_TABLE = (OP == ROPE || OP == LNROPE_FWD || OP == LNROPE_BWD);
    constexpr int DMAX = (OP == LN_FWD || OP == LN_BWD) ? 256 : 128;

    if (!dtype_ok(c.x_dtype)) return RGD_E_DTYPE;
    if (c.B < 0 || c.H < 0 || c.N[0] < 0 || c.N[1] < 0 || c.d < 0) return RGD_E_INVALID;
    if (c.d > DMAX) return RGD_E_SIZE;
    if (c.B > INT32_MAX || c.H > INT32_MAX || c.N[0] > INT32_MAX || c.N[1] > INT32_MAX) return RGD_E_SIZE;
    if (USES_TABLE) {
        if (!(c.pos_dtype == c.x_dtype || c.pos_dtype == RGD_F32)) return RGD_E_DTYPE;
        if (c.R < 0 || c.P < 0) return RGD_E_INVALID;
        // every token index must lie strictly inside the table (head_rope_cached.py:188-189)
        if (!(c.N[0] < c.P) || !(c.N[1] < c.P)) return RGD_E_INVALID;
        if (c.R > 0 && !c.pos) return RGD_E_NULL;
    }
    for (int i = 0; i < 2; ++i) {
        if (!c.x[i] || !c.out[i] || (HAS_DY && !c.dy[i])) return RGD_E_NULL;
        const bool empty = c.B == 0 || c.H == 0 || c.N[i] == 0 || c.d == 0;
        if (!empty && (!c.x[i]->ptr || !c.out[i]->ptr || (HAS_DY && !c.dy[i]->ptr))) return RGD_E_NULL;
    }
    if (c.d == 0 || c.B == 0 || c.H == 0) return RGD_OK;

    const int esize = dtype_size(c.x_dtype);
    const int ve = 16 / esize;
    bool vec = (c.d % ve == 0);
    for (int i = 0; i < 2; ++i) {
        if (c.N[i] == 0) continue;
        vec = vec && heads_vec_ok(*c.x[i], esize) && heads_vec_ok(*c.out[i], esize);
        if (HAS_DY) vec = vec && heads_vec_ok(*c.dy[i], esize);
    }
    // The rotation pairs channels (2i, 2i+1); in vector mode both live in one
    // thread, in scalar mode in neighbouring lanes.
    HeadParams p{};
    int vpt;
    if (vec) {
        const int nvec = (int)c.d / ve;
        int tpr = next_pow2(nvec);
        if (tpr > 32) tpr = 32;
        vpt = (nvec + tpr - 1) / tpr;
        p.tpr = tpr;
    } else {
        p.tpr = 32;
        vpt = ((int)c.d + 31) / 32;
    }
    p.d = (int)c.d;
    p.R = USES_TABLE ? (int)(c.R < c.d ? c.R : c.d) : 0;
    p.pos = c.pos;
    p.pos_ss = c.pos_ss;
    p.pos_sn = c.pos_sn;
    p.transposed = c.transposed;
    p.eps = c.eps;

    const int rows_per_cta = (HEAD_THREADS / p.tpr) * ROWS_PER_THREAD;
    int64_t grid = 0;
    for (int i = 0; i < 2; ++i) {
        HeadTensor &ht = p.t[i];
        const rgd_heads &x = *c.x[i];
        const rgd_heads &o = *c.out[i];
        // Inner dimension = the one with the smaller stride in x.
        const bool seq_inner = (x.stride_n <= x.stride_h);
        ht.seq_inner = seq_inner ? 1 : 0;
        ht.D1 = (int)(seq_inner ? c.H : c.N[i]);
        ht.D2 = (int)(seq_inner ? c.N[i] : c.H);
        ht.x = x.ptr;
        ht.xb = x.stride_b;
        ht.x1 = seq_inner ? x.stride_h : x.stride_n;
        ht.x2 = seq_inner ? x.stride_n : x.stride_h;
        ht.out = o.ptr;
        ht.ob = o.stride_b;
        ht.o1 = seq_inner ? o.stride_h : o.stride_n;
        ht.o2 = seq_inner ? o.stride_n : o.stride_h;
        if (HAS_DY) {
            const rgd_heads &g = *c.dy[i];
            ht.dy = g.ptr;
            ht.db = g.stride_b;
            ht.d1 = seq_inner ? g.stride_h : g.stride_n;
            ht.d2 = seq_inner ? g.stride_n : g.stride_h;
        }
        ht.cut = (int)(c.cut[i] < 0 ? 0 : (c.cut[i] > c.N[i] ? c.N[i] : c.cut[i]));
        ht.rows = c.B * c.H * c.N[i];
        if (ht.D1 == 0) ht.D1 = 1;
        if (ht.D2 == 0) ht.D2 = 1;
        const int64_t ctas = ceil_div64(ht.rows, rows_per_cta);
        if (i == 0) p.split = ctas;
        grid += ctas;
    }
    if (grid == 0) return RGD_OK;
    return dispatch_head<OP>(c, p, vec, vpt, grid, st);
}

}  // namespace
}  // namespace rgd

using namespace rgd;

extern "C" int rgd_headln_fwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *qo, const rgd_heads *ko,
                              int64_t B, int64_t H, int64_t Nq, int64_t Nk, int64_t head_dim, float eps,
                              int dtype, void *stream) {
    HeadCall c{{q, k}, {nullptr, nullptr}, {qo, ko}, B, H, {Nq, Nk}, head_dim, nullptr, 0, 0, 0, 0, {0, 0}, 0, eps,
               dtype, dtype};
    return run_head<LN_FWD>(c, (cudaStream_t)stream);
}

extern "C" int rgd_headln_bwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *dqo, const rgd_heads *dko,
                              const rgd_heads *dq, const rgd_heads *dk, int64_t B, int64_t H, int64_t Nq,
                              int64_t Nk, int64_t head_dim, float eps, int dtype, void *stream) {
    HeadCall c{{q, k}, {dqo, dko}, {dq, dk}, B, H, {Nq, Nk}, head_dim, nullptr, 0, 0, 0, 0, {0, 0}, 0, eps,
               dtype, dtype};
    return run_head<LN_BWD>(c, (cudaStream_t)stream);
}

extern "C" int rgd_rope(const rgd_heads *q, const rgd_heads *k, const void *pos, int64_t pos_stride_s,
                        int64_t pos_stride_n, const rgd_heads *qo, const rgd_heads *ko, int64_t B, int64_t H,
                        int64_t Nq, int64_t Nk, int64_t head_dim, int64_t P, int64_t R, int64_t cut_q,
                        int64_t cut_k, int transposed, int x_dtype, int pos_dtype, void *stream) {
    HeadCall c{{q, k}, {nullptr, nullptr}, {qo, ko}, B, H, {Nq, Nk}, head_dim, pos, pos_stride_s, pos_stride_n,
               P, R, {cut_q, cut_k}, transposed, 0.f, x_dtype, pos_dtype};
    return run_head<ROPE>(c, (cudaStream_t)stream);
}

extern "C" int rgd_lnrope_fwd(const rgd_heads *q, const rgd_heads *k, const void *pos, int64_t pos_stride_s,
                              int64_t pos_stride_n, const rgd_heads *qo, const rgd_heads *ko, int64_t B,
                              int64_t H, int64_t Nq, int64_t Nk, int64_t head_dim, int64_t P, int64_t R,
                              int64_t cut_q, int64_t cut_k, float eps, int x_dtype, int pos_dtype,
                              void *stream) {
    HeadCall c{{q, k}, {nullptr, nullptr}, {qo, ko}, B, H, {Nq, Nk}, head_dim, pos, pos_stride_s, pos_stride_n,
               P, R, {cut_q, cut_k}, 0, eps, x_dtype, pos_dtype};
    return run_head<LNROPE_FWD>(c, (cudaStream_t)stream);
}

extern "C" int rgd_lnrope_bwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *dqo, const rgd_heads *dko,
                              const void *pos, int64_t pos_stride_s, int64_t pos_stride_n, const rgd_heads *dq,
                              const rgd_heads *dk, int64_t B, int64_t H, int64_t Nq, int64_t Nk,
                              int64_t head_dim, int64_t P, int64_t R, int64_t cut_q, int64_t cut_k, float eps,
                              int x_dtype, int pos_dtype, void *stream) {
    HeadCall c{{q, k}, {dqo, dko}, {dq, dk}, B, H, {Nq, Nk}, head_dim, pos, pos_stride_s, pos_stride_n,
               P, R, {cut_q, cut_k}, 0, eps, x_dtype, pos_dtype};
    return run_head<LNROPE_BWD>(c, (cudaStream_t)stream);
}
