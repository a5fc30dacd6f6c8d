// Warp-level building blocks of the general attention kernels: 64-row tiles in
// padded shared memory, ldmatrix fragment loads and m16n8k16 tensor-core MMAs
// with fp32 accumulation.  Used for shapes the tensor-memory kernels do not
// take (head_dim not 64/128, unaligned strides, short sequences).
#pragma once

#include "common.cuh"

namespace rgd {
namespace attn {

constexpr int BM = 64;          // query rows per tile
constexpr int BN = 64;          // key rows per tile
constexpr int NTHREADS = 128;   // 4 warps, 16 tile rows each
constexpr int PAD = 8;          // 16-byte row padding: conflict-free ldmatrix
constexpr float LOG2E = 1.4426950408889634f;
// Internal answer of the tensor-memory entry points: nothing was launched, run the general kernels.
constexpr int TMEM_NOT_TAKEN = -1000;

struct AttnParams {
    const void *q, *k, *v, *o, *d_o;   // (B,H,T,d) views; o / d_o read in the backward
    void *out_o;                       // forward output
    void *dq, *dk, *dv;
    const void *bias;
    float *lse;                        // [B, H, Tq_rounded]
    float *delta;                      // [B, H, Tq_rounded]
    int64_t q_sb, q_sh, q_sn, k_sb, k_sh, k_sn, v_sb, v_sh, v_sn, o_sb, o_sh, o_sn;
    int64_t do_sb, do_sh, do_sn, dq_sb, dq_sh, dq_sn, dk_sb, dk_sh, dk_sn, dv_sb, dv_sh, dv_sn;
    int64_t b_sb, b_sh, b_sq;
    int bias_kind, bias_f32;
    int B, H, Tq, Tk, d, Tq_rounded;
    int causal;
    float scale;
    int vec_q, vec_k, vec_v, vec_o, vec_do, vec_dq, vec_dk, vec_dv;   // 16-byte addressable
    // Bias gradient (backward only), null when not wanted.  Vector bias: fp32 [B, H, Tk], zeroed by
    // the entry point, each key's sum over the queries is added once or twice (the sum of two
    // numbers does not depend on their order).  Matrix bias: [B, H, Tq, Tk] in the tensor dtype
    // through element strides; entries of key blocks a causal mask skips are not written.
    void *dbias;
    int64_t db_sb, db_sh, db_sq;
    int dbias_vec;                     // matrix form: rows are 16-byte addressable
    // Tile lists of a matrix bias (attn_tiles.cu), null when not given: which 128 x 128 tiles are
    // not entirely masked.  Used by the kernels that stage the bias by TMA, without a causal mask.
    const uint16_t *tiles;
};

// Layout of the tile-list buffer of one bias tensor with Bb x Hb distinct (batch, head) slices
// (1 where the bias is broadcast), in 16-bit words from its start; the byte bitmap follows.
//   qcnt [Bb Hb][nqb], qlist [Bb Hb][nqb][nkb]: per 128-query block, the key blocks to visit
//   q2cnt [Bb Hb][nq2], q2list [Bb Hb][nq2][nkb]: the same per 256-query block (union of two)
//   kcnt [Bb Hb][nkb], klist [Bb Hb][nkb][nqb]: per 128-key block, the query blocks to visit
struct TileLayout {
    int64_t slices;
    int nqb, nq2, nkb;
    int64_t qcnt, qlist, q2cnt, q2list, kcnt, klist, words;   // offsets in 16-bit words
    int64_t bitmap_bytes, total_bytes;
};
inline TileLayout tile_layout(int64_t Bb, int64_t Hb, int64_t Tq, int64_t Tk) {
    TileLayout L{};
    L.slices = Bb * Hb;
    L.nqb = (int)((Tq + 127) / 128);
    L.nq2 = (int)((Tq + 255) / 256);
    L.nkb = (int)((Tk + 127) / 128);
    int64_t w = 0;
    L.qcnt = w;   w += L.slices * L.nqb;
    L.qlist = w;  w += L.slices * L.nqb * L.nkb;
    L.q2cnt = w;  w += L.slices * L.nq2;
    L.q2list = w; w += L.slices * L.nq2 * L.nkb;
    L.kcnt = w;   w += L.slices * L.nkb;
    L.klist = w;  w += L.slices * L.nkb * L.nqb;
    L.words = (w + 7) / 8 * 8;
    L.bitmap_bytes = L.slices * L.nqb * L.nkb;
    L.total_bytes = L.words * 2 + (L.bitmap_bytes + 15) / 16 * 16;
    return L;
}

template <typename T> struct Mma;
template <> struct Mma<__half> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct Mma<__nv_bfloat16> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
        asm volatile(
            "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void *smem_row) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void *smem_row) {
    const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

// 64 x DPAD tile of 16-bit elements, rows padded by PAD elements.
template <typename T, int DPAD>
struct Tile {
    static constexpr int LD = DPAD + PAD;
    T data[64 * LD];
    __device__ __forceinline__ T *row(int r) { return data + r * LD; }
    __device__ __forceinline__ const T *row(int r) const { return data + r * LD; }
};

// Fill a tile from global memory: rows [0, rows_valid) x channels [0, d), zero
// elsewhere.  `g` points at (row 0, channel 0); rows are `stride` elements apart.
template <typename T, int DPAD>
__device__ __forceinline__ void load_tile(Tile<T, DPAD> &t, const T *g, int64_t stride, int rows_valid, int d,
                                          bool vec) {
    if (vec) {
        constexpr int CPR = DPAD / 8;
        for (int idx = threadIdx.x; idx < 64 * CPR; idx += NTHREADS) {
            const int r = idx / CPR, c = (idx - r * CPR) * 8;
            uint4 val = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows_valid && c < d) val = *reinterpret_cast<const uint4 *>(g + (int64_t)r * stride + c);
            *reinterpret_cast<uint4 *>(t.row(r) + c) = val;
        }
    } else {
        for (int idx = threadIdx.x; idx < 64 * DPAD; idx += NTHREADS) {
            const int r = idx / DPAD, c = idx - r * DPAD;
            T val = from_f32<T>(0.f);
            if (r < rows_valid && c < d) val = g[(int64_t)r * stride + c];
            t.row(r)[c] = val;
        }
    }
}

// Store a warp's 16 x DPAD fp32 accumulator tile (C-fragment layout) to global
// as T.  `g` points at (tile row 0, channel 0) of this warp's 16 rows.
template <typename T, int DPAD>
__device__ __forceinline__ void store_acc(const float (&acc)[DPAD / 8][4], T *g, int64_t stride, int rows_valid, int d,
                                          bool vec, float scale0, float scale8) {
    const int lane = threadIdx.x & 31, gq = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int nt = 0; nt < DPAD / 8; ++nt) {
        const int c = nt * 8 + 2 * tq;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int r = gq + half * 8;
            const float s = half ? scale8 : scale0;
            const float v0 = acc[nt][half * 2] * s, v1 = acc[nt][half * 2 + 1] * s;
            if (r < rows_valid) {
                T *p = g + (int64_t)r * stride + c;
                if (vec && c + 1 < d) {   // 4-byte aligned: even channel, 8-element-aligned rows
                    *reinterpret_cast<uint32_t *>(p) = Mma<T>::pack(v0, v1);
                } else {
                    if (c < d) p[0] = from_f32<T>(v0);
                    if (c + 1 < d) p[1] = from_f32<T>(v1);
                }
            }
        }
    }
}

// acc[8][4] (16 x 64) += A[16 x DPAD] * B[64 x DPAD]^T, both row-major in shared
// memory (contraction over channels).  a_tile_row0: first of the warp's 16 rows.
template <typename T, int DPAD>
__device__ __forceinline__ void gemm_nt(float (&acc)[8][4], const Tile<T, DPAD> &A, int a_row0,
                                        const Tile<T, DPAD> &B) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < DPAD / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, A.row(a_row0 + (lane & 15)) + kk * 16 + (lane >> 4) * 8);
#pragma unroll
        for (int n2 = 0; n2 < 4; ++n2) {
            uint32_t b[4];
            const int i = lane >> 3;
            ldmatrix_x4(b, B.row(n2 * 16 + (lane & 7) + (i >> 1) * 8) + kk * 16 + (i & 1) * 8);
            Mma<T>::mma(acc[2 * n2], a, b[0], b[1]);
            Mma<T>::mma(acc[2 * n2 + 1], a, b[2], b[3]);
        }
    }
}

// acc[DPAD/8][4] (16 x DPAD) += P[16 x 64] * B[64 x DPAD], P given as packed
// A fragments (p[kk][0..3] for each 16-wide slice of the 64 contraction rows),
// B row-major in shared memory (contraction over its rows).
template <typename T, int DPAD>
__device__ __forceinline__ void gemm_pn(float (&acc)[DPAD / 8][4], const uint32_t (&p)[4][4],
                                        const Tile<T, DPAD> &B) {
    const int lane = threadIdx.x & 31;
    const int i = lane >> 3;
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
        for (int n2 = 0; n2 < DPAD / 16; ++n2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, B.row(kk * 16 + (lane & 7) + (i & 1) * 8) + n2 * 16 + (i >> 1) * 8);
            Mma<T>::mma(acc[2 * n2], p[kk], b[0], b[1]);
            Mma<T>::mma(acc[2 * n2 + 1], p[kk], b[2], b[3]);
        }
    }
}

// Pack a 16 x 64 fp32 C-fragment tile into A fragments of 16-bit values.
template <typename T>
__device__ __forceinline__ void pack_p(uint32_t (&p)[4][4], const float (&s)[8][4]) {
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
        p[kk][0] = Mma<T>::pack(s[2 * kk][0], s[2 * kk][1]);
        p[kk][1] = Mma<T>::pack(s[2 * kk][2], s[2 * kk][3]);
        p[kk][2] = Mma<T>::pack(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        p[kk][3] = Mma<T>::pack(s[2 * kk + 1][2], s[2 * kk + 1][3]);
    }
}

// Bias value for (query i, key j) of this (batch, head); caller guarantees
// i < Tq and j < Tk.
template <typename T>
__device__ __forceinline__ float bias_at_t(const AttnParams &p, const void *bias_bh, int i, int j) {
    const int64_t off = (p.bias_kind == RGD_BIAS_MATRIX ? (int64_t)i * p.b_sq : 0) + j;
    if (p.bias_f32) return reinterpret_cast<const float *>(bias_bh)[off];
    return to_f32<T>(reinterpret_cast<const T *>(bias_bh)[off]);
}

}  // namespace attn
}  // namespace rgd
