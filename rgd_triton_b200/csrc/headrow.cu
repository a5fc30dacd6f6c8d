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

// Fast division of a 31-bit unsigned value by a runtime constant
// (q = umulhi(n, mul) >> shr), precomputed on the host.
struct FastDiv {
    uint32_t mul, shr, div;
};

struct HeadParams {
    HeadTensor t[2];
    int64_t split;      // tiles that belong to tensor 0
    int64_t tiles1;     // tiles that belong to tensor 1
    FastDiv f1[2], f2[2];   // fast divisors by D1 / D2 of each tensor
    int d;              // head_dim
    int tpr;            // threads per row (power of two <= 32)
    int R;              // rotary channels
    const void *pos;    // [2, P, R]: sin, cos
    int64_t pos_ss, pos_sn;
    int transposed;     // rotary: apply the inverse rotation
    int flat;           // every tensor is densely packed rows of d channels in walk order
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

__device__ __forceinline__ uint32_t fdiv(uint32_t n, const FastDiv &f) {
    return f.div == 1 ? n : (__umulhi(n, f.mul) >> f.shr);
}

// Row id -> (batch, outer, inner) indices of a head tensor.
__device__ __forceinline__ void row_index(const HeadTensor &ht, const FastDiv &f1, const FastDiv &f2, int64_t rid,
                                          int64_t &b, int &i1, int &i2) {
    if (ht.rows <= 0x7fffffffLL) {
        const uint32_t r32 = (uint32_t)rid;
        const uint32_t q1 = fdiv(r32, f2);
        i2 = (int)(r32 - q1 * f2.div);
        const uint32_t q2 = fdiv(q1, f1);
        i1 = (int)(q1 - q2 * f1.div);
        b = q2;
    } else {
        i2 = (int)(rid % ht.D2);
        const int64_t q1 = rid / ht.D2;
        i1 = (int)(q1 % ht.D1);
        b = q1 / ht.D1;
    }
}

// Native packed 16-bit arithmetic for the stand-alone rotary on a 16-bit tensor
// with a table of the same type.  The reference evaluates x*cos + rot(x)*sin in
// that type (head_rope_cached.py:48); its compiled kernel contracts the second
// product into the sum, i.e. out = rn(fma(rot, sin, rn(x*cos))) — measured
// bit-equal on B200 — which is what mul + fma below reproduce.
template <typename T> struct Packed2;
template <> struct Packed2<__half> {
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
        __half2 r = __hmul2_rn(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        __half2 r = __hfma2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b),
                            *reinterpret_cast<__half2 *>(&c));
        return *reinterpret_cast<uint32_t *>(&r);
    }
};
template <> struct Packed2<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t b) {
        __nv_bfloat162 r = __hmul2_rn(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b));
        return *reinterpret_cast<uint32_t *>(&r);
    }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t b, uint32_t c) {
        __nv_bfloat162 r = __hfma2(*reinterpret_cast<__nv_bfloat162 *>(&a), *reinterpret_cast<__nv_bfloat162 *>(&b),
                                   *reinterpret_cast<__nv_bfloat162 *>(&c));
        return *reinterpret_cast<uint32_t *>(&r);
    }
};
template <> struct Packed2<float> {   // never used (fp32 tensors take the fp32 path)
    static __device__ __forceinline__ uint32_t mul(uint32_t a, uint32_t) { return a; }
    static __device__ __forceinline__ uint32_t fma(uint32_t a, uint32_t, uint32_t) { return a; }
};

// VE table entries as fp32 from 16-byte words fetched earlier.
template <typename TP, int VE>
__device__ __forceinline__ void table_from_raw(const uint4 *raw, float *out) {
    constexpr int PER = 16 / sizeof(TP);
#pragma unroll
    for (int a = 0; a < (VE + PER - 1) / PER; ++a) {
        union { uint4 u; TP v[PER]; } c;
        c.u = raw[a];
#pragma unroll
        for (int e = 0; e < PER && a * PER + e < VE; ++e) out[a * PER + e] = to_f32<TP>(c.v[e]);
    }
}

// One row: xq (and gq, the upstream gradient) hold this thread's packed slots;
// the result comes back packed in `out`.  T: tensor element type.  TP: table
// element type (T or float).  VE: elements per access (16 / sizeof(T), or 1).
// VPT: column slots per thread.
template <typename T, typename TP, int VE, int VPT, int OP, int DFIX = 0>
__device__ __forceinline__ void process_row(const HeadParams &p, const Vec<T, VE> (&xq)[VPT],
                                            const Vec<T, VE> (&gq)[VPT], int tok, int cut, int t, bool pos_vec_ok,
                                            Vec<T, VE> (&out)[VPT]) {
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    constexpr bool HAS_ROPE = (OP == ROPE || OP == LNROPE_FWD || OP == LNROPE_BWD);
    constexpr bool HAS_LN = (OP != ROPE);
    // The stand-alone rotary computes in the promoted type of x and the table
    // (head_rope_cached.py:48,142): 16-bit x with a 16-bit table rounds x*cos to
    // that type and then fuses rot*sin into the sum; anything else is plain fp32.
    constexpr bool ROUND_EACH = (OP == ROPE) && (sizeof(T) == 2) && (sizeof(TP) == 2);
    constexpr int NE = VPT * VE;
    // DFIX > 0: head_dim is a compile-time constant that fills the slots exactly,
    // so the group width and every bounds check fold away.
    const int tpr = DFIX > 0 ? DFIX / NE : p.tpr;
    const int d = DFIX > 0 ? DFIX : p.d;
    const float invd = 1.0f / (float)d;

    // Rotary tables: fetch the 16-byte words of every fully rotated slot first,
    // so their latency overlaps the normalisation arithmetic below.
    constexpr int TW = (VE * (int)sizeof(TP) + 15) / 16;        // 16-byte words per slot of the table
    const bool rot_row = HAS_ROPE && tok < cut;
    uint4 sraw[HAS_ROPE ? VPT : 1][TW], craw[HAS_ROPE ? VPT : 1][TW];
    bool pre[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
        pre[j] = false;
        if constexpr (HAS_ROPE && VE > 1) {
            const int col = (t + j * tpr) * VE;
            pre[j] = rot_row && pos_vec_ok && col + VE <= p.R;
            if (pre[j]) {
                const TP *srow = reinterpret_cast<const TP *>(p.pos) + (int64_t)tok * p.pos_sn + col;
#pragma unroll
                for (int a = 0; a < TW; ++a) {
                    sraw[j][a] = __ldg(reinterpret_cast<const uint4 *>(srow) + a);
                    craw[j][a] = __ldg(reinterpret_cast<const uint4 *>(srow + p.pos_ss) + a);
                }
            }
        }
    }

    if constexpr (OP == ROPE && ROUND_EACH && VE == 8) {
        // Stand-alone rotary on a 16-bit tensor with a table of the same type: when
        // every slot of this thread is either fully rotated or untouched, evaluate
        // out = fma(rot(x), sin, x*cos) with packed 16-bit instructions (no fp32 round trip).
        bool simple = true;
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int col = (t + j * tpr) * VE;
            if (rot_row && col < p.R && col < d && !pre[j]) simple = false;
        }
        if (simple) {
            const uint32_t flip = sizeof(T) == 2 ? (p.transposed ? 0x80000000u : 0x00008000u) : 0u;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                if (pre[j]) {
                    union { Vec<T, VE> v; uint32_t w[4]; } cx, co;
                    cx.v = xq[j];
                    const uint32_t sw[4] = {sraw[j][0].x, sraw[j][0].y, sraw[j][0].z, sraw[j][0].w};
                    const uint32_t cw[4] = {craw[j][0].x, craw[j][0].y, craw[j][0].z, craw[j][0].w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        // (x_even, x_odd) -> (-x_odd, x_even); the inverse negates the other half
                        const uint32_t rot = __byte_perm(cx.w[i], 0, 0x1032) ^ flip;
                        co.w[i] = Packed2<T>::fma(rot, sw[i], Packed2<T>::mul(cx.w[i], cw[i]));
                    }
                    out[j] = co.v;
                } else {
                    out[j] = xq[j];
                }
            }
            return;
        }
    }

    float xv[NE];
    float dv[HAS_DY ? NE : 1];
#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < VE; ++e) {
            xv[j * VE + e] = to_f32<T>(xq[j].v[e]);
            if constexpr (HAS_DY) dv[j * VE + e] = to_f32<T>(gq[j].v[e]);
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
                const float c = (DFIX > 0 || col < d) ? xv[j * VE + e] - mean : 0.f;
                xv[j * VE + e] = c;           // centred
                s2 += c * c;
            }
        rstd = rsqrtf(warp_group_sum(s2, tpr) * invd + p.eps);
#pragma unroll
        for (int i = 0; i < NE; ++i) xv[i] *= rstd;   // xhat
    }

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
                const TP *srow = reinterpret_cast<const TP *>(p.pos) + (int64_t)tok * p.pos_sn;
                const TP *crow = srow + p.pos_ss;
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const int col = (t + j * tpr) * VE;
                    if (col < p.R) {
                        float sn[VE], cs[VE];
                        if (pre[j]) {
                            table_from_raw<TP, VE>(sraw[j], sn);
                            table_from_raw<TP, VE>(craw[j], cs);
                        } else {
                            load_table<TP, VE>(srow, col, p.R, pos_vec_ok, sn);
                            load_table<TP, VE>(crow, col, p.R, pos_vec_ok, cs);
                        }
                        if constexpr (VE > 1) {
#pragma unroll
                            for (int e = 0; e < VE; e += 2) {
                                const float ge = g[j * VE + e], go = g[j * VE + e + 1];
                                if (pre[j] || col + e < p.R) g[j * VE + e] = ge * cs[e] + go * sn[e];
                                if (pre[j] || col + e + 1 < p.R) g[j * VE + e + 1] = go * cs[e + 1] - ge * sn[e + 1];
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
            const TP *srow = reinterpret_cast<const TP *>(p.pos) + (int64_t)tok * p.pos_sn;
            const TP *crow = srow + p.pos_ss;
            const bool inv = (OP == ROPE) && p.transposed;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int col = (t + j * tpr) * VE;
                if (col < p.R) {
                    float sn[VE], cs[VE];
                    if (pre[j]) {
                        table_from_raw<TP, VE>(sraw[j], sn);
                        table_from_raw<TP, VE>(craw[j], cs);
                    } else {
                        load_table<TP, VE>(srow, col, p.R, pos_vec_ok, sn);
                        load_table<TP, VE>(crow, col, p.R, pos_vec_ok, cs);
                    }
                    if constexpr (VE > 1) {
#pragma unroll
                        for (int e = 0; e < VE; e += 2) {
                            const float xe = xv[j * VE + e], xo = xv[j * VE + e + 1];
                            // rotated partner: (-x_odd, x_even), sign flipped for the inverse
                            const float re = inv ? xo : -xo;
                            const float ro = inv ? -xe : xe;
                            float oe, oo;
                            if constexpr (ROUND_EACH) {
                                // rot*sin is exact in fp32 for 16-bit operands
                                oe = round_to<T>(fmaf(re, sn[e], round_to<T>(xe * cs[e])));
                                oo = round_to<T>(fmaf(ro, sn[e + 1], round_to<T>(xo * cs[e + 1])));
                            } else {
                                oe = xe * cs[e] + re * sn[e];
                                oo = xo * cs[e + 1] + ro * sn[e + 1];
                            }
                            if (pre[j] || col + e < p.R) res[j * VE + e] = oe;
                            if (pre[j] || col + e + 1 < p.R) res[j * VE + e + 1] = oo;
                        }
                    } else {
                        const float me = xv[j];
                        float rot = (col & 1) ? oth[j] : -oth[j];
                        if (inv) rot = -rot;
                        if constexpr (ROUND_EACH)
                            res[j] = round_to<T>(fmaf(rot, sn[0], round_to<T>(me * cs[0])));
                        else
                            res[j] = me * cs[0] + rot * sn[0];
                    }
                }
            }
        }
    }


#pragma unroll
    for (int j = 0; j < VPT; ++j)
#pragma unroll
        for (int e = 0; e < VE; ++e) out[j].v[e] = from_f32<T>(res[j * VE + e]);
}

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)),
                 "l"(gsrc)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Direct kernel: one tile (rows-per-CTA x ROWS_PER_THREAD rows) per CTA, loads
// straight into registers.  Used for rows that are not 16-byte addressable.
template <typename T, typename TP, int VE, int VPT, int OP>
__global__ void __launch_bounds__(HEAD_THREADS) head_kernel(const __grid_constant__ HeadParams p) {
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    using V = Vec<T, VE>;

    const int ti = (int64_t)blockIdx.x >= p.split ? 1 : 0;
    const HeadTensor &ht = p.t[ti];
    const int64_t local = (int64_t)blockIdx.x - (ti ? p.split : 0);
    const int tpr = p.tpr;
    const int rpc = HEAD_THREADS / tpr;                 // rows per CTA pass
    const int rg = (int)threadIdx.x / tpr;
    const int t = (int)threadIdx.x - rg * tpr;
    const int d = p.d;
    const bool pos_vec_ok = (reinterpret_cast<uintptr_t>(p.pos) % 16 == 0) &&
                            (p.pos_ss % (16 / (int)sizeof(TP)) == 0) && (p.pos_sn % (16 / (int)sizeof(TP)) == 0);

#pragma unroll 1
    for (int r = 0; r < ROWS_PER_THREAD; ++r) {
        const int64_t rid = (local * ROWS_PER_THREAD + r) * rpc + rg;
        const bool valid = rid < ht.rows;
        int64_t b;
        int i1, i2;
        row_index(ht, p.f1[ti], p.f2[ti], valid ? rid : 0, b, i1, i2);
        const int tok = ht.seq_inner ? i2 : i1;
        const T *xr = reinterpret_cast<const T *>(ht.x) + b * ht.xb + (int64_t)i1 * ht.x1 + (int64_t)i2 * ht.x2;
        const T *dr = HAS_DY ? reinterpret_cast<const T *>(ht.dy) + b * ht.db + (int64_t)i1 * ht.d1 + (int64_t)i2 * ht.d2
                             : nullptr;
        V xq[VPT], gq[VPT], res[VPT];
#pragma unroll
        for (int j = 0; j < VPT; ++j) {
            const int col = (t + j * tpr) * VE;
            if (valid && col < d) {
                xq[j] = load_vec<T, VE>(xr + col);
                if constexpr (HAS_DY) gq[j] = load_vec<T, VE>(dr + col);
            } else {
#pragma unroll
                for (int e = 0; e < VE; ++e) {
                    xq[j].v[e] = from_f32<T>(0.f);
                    gq[j].v[e] = from_f32<T>(0.f);
                }
            }
        }
        process_row<T, TP, VE, VPT, OP>(p, xq, gq, tok, ht.cut, t, pos_vec_ok, res);
        if (valid) {
            T *orow = reinterpret_cast<T *>(ht.out) + b * ht.ob + (int64_t)i1 * ht.o1 + (int64_t)i2 * ht.o2;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int col = (t + j * tpr) * VE;
                if (col < d) store_vec<T, VE>(orow + col, res[j]);
            }
        }
    }
}

// Pipelined kernel for 16-byte addressable rows: persistent CTAs walk the tiles
// of both tensors; the 16-byte pieces of the next PIPE_STAGES-1 tiles are in
// flight (cp.async) into per-thread shared-memory slots while the current tile
// is normalised / rotated from registers and stored with streaming stores.
// Each thread reads back only the slots it filled itself, so no block-level
// barrier is needed; cp.async.wait_group orders a thread's own copies.
constexpr int PIPE_STAGES = 3;

template <typename T, typename TP, int VPT, int OP>
__global__ void __launch_bounds__(HEAD_THREADS) head_kernel_pipelined(const __grid_constant__ HeadParams p) {
    constexpr int VE = VecElems<T>::value;
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    constexpr int NIN = HAS_DY ? 2 : 1;
    constexpr int SLOTS = NIN * ROWS_PER_THREAD * VPT;   // 16-byte slots per thread and stage
    using V = Vec<T, VE>;
    extern __shared__ uint4 slots[];                     // [PIPE_STAGES][SLOTS][HEAD_THREADS]

    const int tpr = p.tpr;
    const int rpc = HEAD_THREADS / tpr;
    const int rg = (int)threadIdx.x / tpr;
    const int t = (int)threadIdx.x - rg * tpr;
    const int d = p.d;
    const int64_t total = p.split + p.tiles1;
    const bool pos_vec_ok = (reinterpret_cast<uintptr_t>(p.pos) % 16 == 0) &&
                            (p.pos_ss % (16 / (int)sizeof(TP)) == 0) && (p.pos_sn % (16 / (int)sizeof(TP)) == 0);
    auto slot = [&](int stage, int idx) -> uint4 * {
        return slots + ((size_t)stage * SLOTS + idx) * HEAD_THREADS + threadIdx.x;
    };

    auto issue = [&](int64_t tile, int stage) {
        const int ti = tile >= p.split ? 1 : 0;
        const HeadTensor &ht = p.t[ti];
        const int64_t local = tile - (ti ? p.split : 0);
#pragma unroll
        for (int r = 0; r < ROWS_PER_THREAD; ++r) {
            const int64_t rid = (local * ROWS_PER_THREAD + r) * rpc + rg;
            const bool valid = rid < ht.rows;
            int64_t b;
            int i1, i2;
            row_index(ht, p.f1[ti], p.f2[ti], valid ? rid : 0, b, i1, i2);
            const T *xr = reinterpret_cast<const T *>(ht.x) + b * ht.xb + (int64_t)i1 * ht.x1 + (int64_t)i2 * ht.x2;
            const T *dr = HAS_DY ? reinterpret_cast<const T *>(ht.dy) + b * ht.db + (int64_t)i1 * ht.d1 +
                                       (int64_t)i2 * ht.d2
                                 : nullptr;
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int col = (t + j * tpr) * VE;
                if (valid && col < d) {
                    cp_async16(slot(stage, r * VPT + j), xr + col);
                    if constexpr (HAS_DY) cp_async16(slot(stage, (ROWS_PER_THREAD + r) * VPT + j), dr + col);
                }
            }
        }
    };

    auto consume = [&](int64_t tile, int stage) {
        const int ti = tile >= p.split ? 1 : 0;
        const HeadTensor &ht = p.t[ti];
        const int64_t local = tile - (ti ? p.split : 0);
#pragma unroll
        for (int r = 0; r < ROWS_PER_THREAD; ++r) {
            const int64_t rid = (local * ROWS_PER_THREAD + r) * rpc + rg;
            const bool valid = rid < ht.rows;
            int64_t b;
            int i1, i2;
            row_index(ht, p.f1[ti], p.f2[ti], valid ? rid : 0, b, i1, i2);
            const int tok = ht.seq_inner ? i2 : i1;
            V xq[VPT], gq[VPT], res[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                const int col = (t + j * tpr) * VE;
                union { uint4 u; V v; } cx, cg;
                cx.u = make_uint4(0u, 0u, 0u, 0u);
                cg.u = make_uint4(0u, 0u, 0u, 0u);
                if (valid && col < d) {
                    cx.u = *slot(stage, r * VPT + j);
                    if constexpr (HAS_DY) cg.u = *slot(stage, (ROWS_PER_THREAD + r) * VPT + j);
                }
                xq[j] = cx.v;
                gq[j] = cg.v;
            }
            process_row<T, TP, VE, VPT, OP>(p, xq, gq, tok, ht.cut, t, pos_vec_ok, res);
            if (valid) {
                T *orow = reinterpret_cast<T *>(ht.out) + b * ht.ob + (int64_t)i1 * ht.o1 + (int64_t)i2 * ht.o2;
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    const int col = (t + j * tpr) * VE;
                    if (col < d) store_vec_stream<T, VE>(orow + col, res[j]);
                }
            }
        }
    };

    const int64_t step = gridDim.x;
    const int64_t tile0 = blockIdx.x;
#pragma unroll
    for (int s = 0; s < PIPE_STAGES - 1; ++s) {
        if (tile0 + s * step < total) issue(tile0 + s * step, s);
        cp_async_commit();
    }
    int stage = 0;
    for (int64_t tile = tile0; tile < total; tile += step) {
        const int64_t ahead = tile + (PIPE_STAGES - 1) * step;
        int fill = stage + PIPE_STAGES - 1;
        if (fill >= PIPE_STAGES) fill -= PIPE_STAGES;
        if (ahead < total) issue(ahead, fill);
        cp_async_commit();
        cp_async_wait<PIPE_STAGES - 1>();      // this thread's copies for `tile` have landed
        consume(tile, stage);
        if (++stage == PIPE_STAGES) stage = 0;
    }
    cp_async_wait<0>();
}

// Flat kernel: the common case of densely packed tensors (x, dy and out are all
// [rows, D] with pitch D in the same row order) and head_dim D known at compile
// time.  Row r lives at base + r * D, so the per-row address arithmetic is one
// multiply-add and the token index one or two fast divisions.  Same persistent
// cp.async pipeline as head_kernel_pipelined.
// Geometry of the flat kernel (16-byte slots per thread-row, rows per thread), chosen by
// measurement: forward operators run best with a quarter row per thread (fewer shuffle
// rounds and index computations per byte), the backward ones, which hold x and dy, with
// an eighth of a row and two rows in flight.
template <int OP> struct FlatGeom {
    static constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    static constexpr int VPT = HAS_DY ? 2 : 4;
    static constexpr int RPT = HAS_DY ? 2 : 1;
    // The backward operators are bound by instruction issue with long dependent chains (four
    // row reductions): a third CTA per SM (80 registers, two pipeline stages instead of three so
    // that the shared memory fits) hides them better (LayerNorm+rotary backward 167 -> 155 us at
    // the second benchmark configuration).  The forward operators lose by the same trade.
    static constexpr int STAGES = HAS_DY ? 2 : PIPE_STAGES;
    static constexpr int MIN_CTAS = HAS_DY ? 3 : 0;      // 0: no constraint for the forward operators
};

template <typename T, typename TP, int VPT, int FLAT_RPT, int OP, int D>
__global__ void __launch_bounds__(HEAD_THREADS, FlatGeom<OP>::MIN_CTAS) head_kernel_flat(const __grid_constant__ HeadParams p) {
    constexpr int VE = VecElems<T>::value;
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    constexpr bool HAS_ROPE = (OP == ROPE || OP == LNROPE_FWD || OP == LNROPE_BWD);
    constexpr int NIN = HAS_DY ? 2 : 1;
    constexpr int TPR = D / (VE * VPT);                  // threads per row
    constexpr int RPC = HEAD_THREADS / TPR;              // rows per CTA pass
    constexpr int SLOTS = NIN * FLAT_RPT * VPT;
    constexpr int STAGES = FlatGeom<OP>::STAGES;
    using V = Vec<T, VE>;
    extern __shared__ uint4 slots[];                     // [STAGES][SLOTS][HEAD_THREADS]

    const int rg = (int)threadIdx.x / TPR;
    const int t = (int)threadIdx.x - rg * TPR;
    const int64_t total = p.split + p.tiles1;
    const bool pos_vec_ok = (reinterpret_cast<uintptr_t>(p.pos) % 16 == 0) &&
                            (p.pos_ss % (16 / (int)sizeof(TP)) == 0) && (p.pos_sn % (16 / (int)sizeof(TP)) == 0);
    auto slot = [&](int stage, int idx) -> uint4 * {
        return slots + ((size_t)stage * SLOTS + idx) * HEAD_THREADS + threadIdx.x;
    };

    auto issue = [&](int64_t tile, int stage) {
        const int ti = tile >= p.split ? 1 : 0;
        const HeadTensor &ht = p.t[ti];
        const int64_t row0 = (tile - (ti ? p.split : 0)) * (FLAT_RPT * RPC) + rg;
        const T *xb = reinterpret_cast<const T *>(ht.x) + t * VE;
        const T *gb = HAS_DY ? reinterpret_cast<const T *>(ht.dy) + t * VE : nullptr;
#pragma unroll
        for (int r = 0; r < FLAT_RPT; ++r) {
            const int64_t rid = row0 + r * RPC;
            if (rid < ht.rows) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) {
                    cp_async16(slot(stage, r * VPT + j), xb + rid * D + j * TPR * VE);
                    if constexpr (HAS_DY)
                        cp_async16(slot(stage, (FLAT_RPT + r) * VPT + j), gb + rid * D + j * TPR * VE);
                }
            }
        }
    };

    auto consume = [&](int64_t tile, int stage) {
        const int ti = tile >= p.split ? 1 : 0;
        const HeadTensor &ht = p.t[ti];
        const int64_t row0 = (tile - (ti ? p.split : 0)) * (FLAT_RPT * RPC) + rg;
        T *ob = reinterpret_cast<T *>(ht.out) + t * VE;
        const FastDiv f2 = p.f2[ti], f1 = p.f1[ti];
#pragma unroll
        for (int r = 0; r < FLAT_RPT; ++r) {
            const int64_t rid = row0 + r * RPC;
            const bool valid = rid < ht.rows;
            int tok = 0;
            if constexpr (HAS_ROPE) {
                // token index of the row: rows are (batch, outer, inner)-major
                const uint32_t r32 = (uint32_t)(valid ? rid : 0);
                const uint32_t q1 = fdiv(r32, f2);
                if (ht.seq_inner) {
                    tok = (int)(r32 - q1 * f2.div);
                } else {
                    const uint32_t q2 = fdiv(q1, f1);
                    tok = (int)(q1 - q2 * f1.div);
                }
            }
            V xq[VPT], gq[VPT], res[VPT];
#pragma unroll
            for (int j = 0; j < VPT; ++j) {
                union { uint4 u; V v; } cx, cg;
                cx.u = make_uint4(0u, 0u, 0u, 0u);
                cg.u = make_uint4(0u, 0u, 0u, 0u);
                if (valid) {
                    cx.u = *slot(stage, r * VPT + j);
                    if constexpr (HAS_DY) cg.u = *slot(stage, (FLAT_RPT + r) * VPT + j);
                }
                xq[j] = cx.v;
                gq[j] = cg.v;
            }
            process_row<T, TP, VE, VPT, OP, D>(p, xq, gq, tok, ht.cut, t, pos_vec_ok, res);
            if (valid) {
#pragma unroll
                for (int j = 0; j < VPT; ++j) store_vec_stream<T, VE>(ob + rid * D + j * TPR * VE, res[j]);
            }
        }
    };

    const int64_t step = gridDim.x;
    const int64_t tile0 = blockIdx.x;
#pragma unroll
    for (int s = 0; s < STAGES - 1; ++s) {
        if (tile0 + s * step < total) issue(tile0 + s * step, s);
        cp_async_commit();
    }
    int stage = 0;
    for (int64_t tile = tile0; tile < total; tile += step) {
        const int64_t ahead = tile + (STAGES - 1) * step;
        int fill = stage + STAGES - 1;
        if (fill >= STAGES) fill -= STAGES;
        if (ahead < total) issue(ahead, fill);
        cp_async_commit();
        cp_async_wait<STAGES - 1>();
        consume(tile, stage);
        if (++stage == STAGES) stage = 0;
    }
    cp_async_wait<0>();
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

FastDiv make_fastdiv(uint32_t d) {
    FastDiv f{0, 0, d};
    if (d <= 1) return f;
    uint32_t lg = 0;
    while ((1ull << lg) < d) ++lg;                 // ceil(log2 d)
    const uint32_t pw = 31 + lg;
    f.mul = (uint32_t)(((1ull << pw) + d - 1) / d);
    f.shr = pw - 32;
    return f;
}

template <typename T, typename TP, int VPT, int OP>
int launch_pipelined(const HeadParams &p, int64_t tiles, cudaStream_t st) {
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    constexpr int SLOTS = (HAS_DY ? 2 : 1) * ROWS_PER_THREAD * VPT;
    const size_t smem = (size_t)PIPE_STAGES * SLOTS * HEAD_THREADS * 16;
    auto kernel = head_kernel_pipelined<T, TP, VPT, OP>;
    if (smem > 32 * 1024)   // static shared memory counts towards the 48 KB default limit too
        if (int e = ensure_dyn_smem(reinterpret_cast<const void *>(kernel), smem)) return e;
    // Persistent grid, never more CTAs than tiles:
    // one resident wave of persistent CTAs
    const int per_sm = cached_occupancy(reinterpret_cast<const void *>(kernel), HEAD_THREADS, smem);
    int64_t grid = (int64_t)num_sms() * per_sm;
    if (grid > tiles) grid = tiles;
    kernel<<<(unsigned)grid, HEAD_THREADS, smem, st>>>(p);
    count_launch();
    return check_launch();
}

template <typename T, typename TP, int OP, int D>
int launch_flat(const HeadParams &p, int64_t tiles, cudaStream_t st) {
    constexpr bool HAS_DY = (OP == LN_BWD || OP == LNROPE_BWD);
    constexpr int VPT = FlatGeom<OP>::VPT, RPT = FlatGeom<OP>::RPT;
    constexpr int SLOTS = (HAS_DY ? 2 : 1) * RPT * VPT;
    const size_t smem = (size_t)FlatGeom<OP>::STAGES * SLOTS * HEAD_THREADS * 16;
    auto kernel = head_kernel_flat<T, TP, VPT, RPT, OP, D>;
    if (smem > 32 * 1024)
        if (int e = ensure_dyn_smem(reinterpret_cast<const void *>(kernel), smem)) return e;
    // one resident wave of persistent CTAs
    const int per_sm = cached_occupancy(reinterpret_cast<const void *>(kernel), HEAD_THREADS, smem);
    int64_t grid = (int64_t)num_sms() * per_sm;
    if (grid > tiles) grid = tiles;
    kernel<<<(unsigned)grid, HEAD_THREADS, smem, st>>>(p);
    count_launch();
    return check_launch();
}

template <typename T, typename TP, int OP>
int launch_head(const HeadParams &p, bool vec, int vpt, int64_t grid, cudaStream_t st) {
    if (grid > INT32_MAX) return RGD_E_SIZE;
    if (p.flat && (p.d == 64 || p.d == 128)) {
        // tiles were counted for p.tpr threads per row; recount for the flat geometry
        constexpr int VE = VecElems<T>::value;
        int64_t tiles[2];
        HeadParams q = p;
        for (int i = 0; i < 2; ++i) {
            const int rows_per_tile = (HEAD_THREADS / (p.d / (VE * FlatGeom<OP>::VPT))) * FlatGeom<OP>::RPT;
            tiles[i] = ceil_div64(p.t[i].rows, rows_per_tile);
        }
        q.split = tiles[0];
        q.tiles1 = tiles[1];
        if (p.d == 128) return launch_flat<T, TP, OP, 128>(q, tiles[0] + tiles[1], st);
        return launch_flat<T, TP, OP, 64>(q, tiles[0] + tiles[1], st);
    }
    if (vec) {
        if (vpt == 1) return launch_pipelined<T, TP, 1, OP>(p, grid, st);
        if (vpt == 2) return launch_pipelined<T, TP, 2, OP>(p, grid, st);
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
    bool all_flat = vec && (c.d * esize) % (16 * FlatGeom<OP>::VPT) == 0;
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
        {
            // dense [B][D1][D2][d] in walk order, for x, out and (backward) dy alike
            auto dense = [&](int64_t sb, int64_t s1, int64_t s2) {
                return s2 == c.d && s1 == (int64_t)ht.D2 * c.d && sb == (int64_t)ht.D1 * ht.D2 * c.d;
            };
            bool f = dense(ht.xb, ht.x1, ht.x2) && dense(ht.ob, ht.o1, ht.o2) && ht.rows <= 0x7fffffffLL;
            if (HAS_DY) f = f && dense(ht.db, ht.d1, ht.d2);
            if (c.N[i] > 0 && !f) all_flat = false;
        }
        p.f1[i] = make_fastdiv((uint32_t)ht.D1);
        p.f2[i] = make_fastdiv((uint32_t)ht.D2);
        const int64_t ctas = ceil_div64(ht.rows, rows_per_cta);
        if (i == 0) p.split = ctas; else p.tiles1 = ctas;
        grid += ctas;
    }
    if (grid == 0) return RGD_OK;
    p.flat = all_flat ? 1 : 0;
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
