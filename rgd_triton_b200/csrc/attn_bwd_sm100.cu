// FlashAttention backward on Blackwell tensor memory (tcgen05 + TMEM + TMA).
//
// Two launches of one kernel template, each producing its outputs in a fixed
// order with no atomics (bit-reproducible, no fp32 dQ scratch):
//   DKDV = true   one CTA per 128 keys, loops over 128-query blocks.  The score
//                 tile is kept TRANSPOSED (keys x queries): G1 = K Q^T,
//                 G2 = V dO^T, so P^T and dS^T land in tensor memory with keys
//                 on the lanes and feed dV += P^T dO and dK += dS^T Q directly
//                 as the tensor-memory A operand.
//   DKDV = false  one CTA per 128 queries, loops over 128-key blocks:
//                 G1 = Q K^T, G2 = dO V^T, dQ += dS K.
// Per block: P = 2^(G1*scale*log2e + bias*log2e - lse*log2e), dS = P (G2 - delta)
// scale; P and dS are rounded to the tensor dtype before their GEMMs, as in
// flash_attn_triton_cached.py:476-522.
//
// Warp roles: warps 0-7 compute (thread = one tile row, half of its 128
// columns; each half packs its 16-bit P / dS into the first 32 of its own 64
// columns, so a thread only ever overwrites columns it has consumed itself),
// warp 8 TMA producer, warp 9 MMA issuer.  Tensor memory: G1 / P in
// columns [0,128), G2 / dS in [128,256), accumulators at 256 and 384.  The MMA
// issue order is software-pipelined — G1 of block i+1 is issued between the two
// accumulation GEMMs of block i — so the exponentials of the next block overlap
// the tensor-core work of the current one.  All waits are bounded.
#include <math.h>

#include "attn_mma.cuh"
#include "sm100_prims.cuh"

namespace rgd {
namespace attn {

using namespace rgd::sm100;

int *tmem_status_ptr();   // attn_fwd_sm100.cu

constexpr int BWD_THREADS = 320;
constexpr int BT = 128;   // tile edge (queries and keys)

struct BwdTmaParams {
    CUtensorMap mq, mk, mv, mdo;
    void *out1, *out2;                  // DKDV: dV, dK.  DQ: dQ, unused.
    int64_t o1_sb, o1_sh, o1_sn, o2_sb, o2_sh, o2_sn;
    const void *bias;
    int64_t b_sb, b_sh, b_sq;
    int bias_kind, bias_f32, bias_vec;
    const float *lse, *delta;           // [B, H, Tq_rounded]
    int H, Tq, Tk, Tq_rounded, causal;
    float scale, scale_log2;
    int *status;
};

template <int D>
struct alignas(1024) BwdTmaSmem {
    unsigned char x1[BT * D * 2], x2[BT * D * 2];            // fixed tiles
    unsigned char y1[2][BT * D * 2], y2[2][BT * D * 2];      // looped tiles, 2 stages
    uint64_t x_full, g1_full, g2_full, p_ready, ds_ready, acc_full;
    uint64_t y_full[2], y_empty[2];
    uint32_t tmem_base;
};

__device__ __forceinline__ float ex2b(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
template <bool BF16>
__device__ __forceinline__ uint32_t pack16b(float a, float b) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    } else {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
}

template <int D, bool BF16, bool DKDV>
__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_tmem(const __grid_constant__ BwdTmaParams p) {
    constexpr int HALVES = D / 64;
    constexpr uint32_t PANEL = 128 * 64 * 2;
    constexpr uint32_t TILE_BYTES = BT * D * 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t G1_COL = 0, G2_COL = 128, ACC1_COL = 256, ACC2_COL = 384;
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;

    extern __shared__ unsigned char smem_raw[];
    BwdTmaSmem<D> &sm = *reinterpret_cast<BwdTmaSmem<D> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int r0 = blk * BT;                               // first key (DKDV) or query (DQ) of this CTA
    // Range of looped blocks.
    int i_begin, i_end;
    if (DKDV) {
        i_begin = p.causal ? r0 / BT : 0;                  // queries before this key block see none of it
        i_end = (p.Tq + BT - 1) / BT;
    } else {
        i_begin = 0;
        i_end = ((p.causal ? min(p.Tk, r0 + BT) : p.Tk) + BT - 1) / BT;
    }
    const int nit = max(i_end - i_begin, 0);
    int *status = p.status;

    if (threadIdx.x == 0) {
        mbar_init(&sm.x_full, 1);
        mbar_init(&sm.g1_full, 1);
        mbar_init(&sm.g2_full, 1);
        mbar_init(&sm.p_ready, 256);
        mbar_init(&sm.ds_ready, 256);
        mbar_init(&sm.acc_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.y_full[s], 1);
            mbar_init(&sm.y_empty[s], 1);
        }
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(&sm.tmem_base, TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tbase = sm.tmem_base;

    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && nit > 0) {
            const CUtensorMap *mx1 = DKDV ? &p.mk : &p.mq, *mx2 = DKDV ? &p.mv : &p.mdo;
            const CUtensorMap *my1 = DKDV ? &p.mq : &p.mk, *my2 = DKDV ? &p.mdo : &p.mv;
            tma_prefetch_desc(mx1);
            tma_prefetch_desc(mx2);
            tma_prefetch_desc(my1);
            tma_prefetch_desc(my2);
            mbar_expect_tx(&sm.x_full, 2 * TILE_BYTES);
            for (int hh = 0; hh < HALVES; ++hh) {
                tma_load_4d(sm.x1 + hh * PANEL, mx1, &sm.x_full, hh * 64, r0, h, b);
                tma_load_4d(sm.x2 + hh * PANEL, mx2, &sm.x_full, hh * 64, r0, h, b);
            }
            bool ok = true;
            for (int it = 0; it < nit; ++it) {
                const int s = it & 1;
                const uint32_t ph = (uint32_t)(it >> 1) & 1u;
                ok = mbar_wait(&sm.y_empty[s], ph ^ 1u, status, 41);
                if (!ok) break;
                mbar_expect_tx(&sm.y_full[s], 2 * TILE_BYTES);
                const int row = (i_begin + it) * BT;
                for (int hh = 0; hh < HALVES; ++hh) {
                    tma_load_4d(sm.y1[s] + hh * PANEL, my1, &sm.y_full[s], hh * 64, row, h, b);
                    tma_load_4d(sm.y2[s] + hh * PANEL, my2, &sm.y_full[s], hh * 64, row, h, b);
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 9) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0 && nit > 0) {
            constexpr uint32_t idesc_g = make_idesc(BF16, BT, BT, false, false);
            constexpr uint32_t idesc_acc = make_idesc(BF16, BT, D, false, true);
            const uint32_t x1a = smem_u32(sm.x1), x2a = smem_u32(sm.x2);
            auto issue_g = [&](uint32_t col, uint32_t xa, uint32_t ya) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * PANEL + (kk % 4) * 32;
                    umma_ss(tbase + col, make_sdesc(xa + off, 16, 1024), make_sdesc(ya + off, 16, 1024), idesc_g, kk > 0);
                }
            };
            auto issue_acc = [&](uint32_t acc_col, uint32_t a_col, uint32_t ya, bool first) {
#pragma unroll
                for (int kk = 0; kk < BT / 16; ++kk)
                    umma_ts(tbase + acc_col, tbase + a_col + (kk >> 2) * 64 + (kk & 3) * 8,
                            make_sdesc(ya + kk * 2048, PANEL, 1024), idesc_acc, !first || kk > 0);
            };
            bool ok = mbar_wait(&sm.x_full, 0, status, 51);
            if (ok) ok = mbar_wait(&sm.y_full[0], 0, status, 52);
            if (ok) {
                tc_fence_after_sync();
                issue_g(G1_COL, x1a, smem_u32(sm.y1[0]));
                umma_commit(&sm.g1_full);
                issue_g(G2_COL, x2a, smem_u32(sm.y2[0]));
                umma_commit(&sm.g2_full);
            }
            for (int it = 0; it < nit && ok; ++it) {
                const int s = it & 1, sn = s ^ 1;
                const uint32_t par = (uint32_t)it & 1u;
                ok = mbar_wait(&sm.p_ready, par, status, 53);
                if (!ok) break;
                tc_fence_after_sync();
                if (DKDV) issue_acc(ACC1_COL, G1_COL, smem_u32(sm.y2[s]), it == 0);     // dV += P^T dO
                const bool more = it + 1 < nit;
                if (more) {
                    ok = mbar_wait(&sm.y_full[sn], (uint32_t)((it + 1) >> 1) & 1u, status, 54);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_g(G1_COL, x1a, smem_u32(sm.y1[sn]));
                    umma_commit(&sm.g1_full);
                }
                ok = mbar_wait(&sm.ds_ready, par, status, 55);
                if (!ok) break;
                tc_fence_after_sync();
                issue_acc(DKDV ? ACC2_COL : ACC1_COL, G2_COL, smem_u32(sm.y1[s]), it == 0);   // dK += dS^T Q | dQ += dS K
                umma_commit(&sm.y_empty[s]);
                if (more) {
                    issue_g(G2_COL, x2a, smem_u32(sm.y2[sn]));
                    umma_commit(&sm.g2_full);
                }
            }
            umma_commit(&sm.acc_full);
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        const int row_l = (warp & 3) * 32 + lane;          // tile row == TMEM lane
        const int half = warp >> 2;                        // which 64 of the 128 columns
        const int row = r0 + row_l;                        // key (DKDV) or query (DQ) index
        const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        const float *lse_bh = p.lse + (int64_t)bh * p.Tq_rounded;
        const float *delta_bh = p.delta + (int64_t)bh * p.Tq_rounded;
        const char *bias_bh = nullptr;
        if (p.bias_kind != RGD_BIAS_NONE)
            bias_bh = reinterpret_cast<const char *>(p.bias) +
                      ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : 2);

        float lse_row = INFINITY, delta_row = 0.f;         // DQ: per-thread row statistics
        if (!DKDV && row < p.Tq) {
            lse_row = lse_bh[row] * LOG2E;
            delta_row = delta_bh[row];
        }

        bool ok = true;
        for (int it = 0; it < nit; ++it) {
            const uint32_t par = (uint32_t)it & 1u;
            const int c0 = (i_begin + it) * BT + half * 64;   // first column index (query for DKDV, key for DQ)
            float pv[64];

            ok = mbar_wait(&sm.g1_full, par, status, 61);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                tmem_ld32(lane_base + G1_COL + half * 64 + c * 32, r);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int col = c0 + c * 32 + i;
                    const int qi = DKDV ? col : row, kj = DKDV ? row : col;
                    float x = __uint_as_float(r[i]) * p.scale_log2;
                    const bool masked = kj >= p.Tk || qi >= p.Tq || (p.causal && kj > qi);
                    float l2;
                    if (DKDV) l2 = (qi < p.Tq) ? __ldg(lse_bh + qi) * LOG2E : INFINITY;
                    else l2 = lse_row;
                    if (bias_bh != nullptr && !masked) {
                        const int64_t off = (p.bias_kind == RGD_BIAS_MATRIX ? (int64_t)qi * p.b_sq : 0) + kj;
                        x += (p.bias_f32 ? reinterpret_cast<const float *>(bias_bh)[off]
                                         : to_f32<T>(reinterpret_cast<const T *>(bias_bh)[off])) * LOG2E;
                    }
                    pv[c * 32 + i] = masked ? 0.f : ex2b(x - l2);
                }
                if (DKDV) {
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) pk[i] = pack16b<BF16>(pv[c * 32 + 2 * i], pv[c * 32 + 2 * i + 1]);
                    tmem_st16(lane_base + G1_COL + half * 64 + c * 16, pk);
                }
            }
            if (DKDV) tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.p_ready);

            ok = mbar_wait(&sm.g2_full, par, status, 62);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t g2[32];
                tmem_ld32(lane_base + G2_COL + half * 64 + c * 32, g2);
                tmem_wait_ld();
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float d0, d1;
                    if (DKDV) {
                        const int q0 = c0 + c * 32 + i;
                        d0 = (q0 < p.Tq) ? __ldg(delta_bh + q0) : 0.f;
                        d1 = (q0 + 1 < p.Tq) ? __ldg(delta_bh + q0 + 1) : 0.f;
                    } else {
                        d0 = d1 = delta_row;
                    }
                    const float s0 = pv[c * 32 + i] * (__uint_as_float(g2[i]) - d0) * p.scale;
                    const float s1 = pv[c * 32 + i + 1] * (__uint_as_float(g2[i + 1]) - d1) * p.scale;
                    pk[i >> 1] = pack16b<BF16>(s0, s1);
                }
                tmem_st16(lane_base + G2_COL + half * 64 + c * 16, pk);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.ds_ready);
        }

        // epilogue: accumulators -> global
        if (ok && nit > 0) ok = mbar_wait(&sm.acc_full, 0, status, 63);
        tc_fence_after_sync();
        if (ok) {
            const int limit = DKDV ? p.Tk : p.Tq;
            constexpr int NOUT = DKDV ? 2 : 1;
#pragma unroll
            for (int o = 0; o < NOUT; ++o) {
                T *base = reinterpret_cast<T *>(o == 0 ? p.out1 : p.out2);
                const int64_t sb = o == 0 ? p.o1_sb : p.o2_sb, sh = o == 0 ? p.o1_sh : p.o2_sh,
                              sn = o == 0 ? p.o1_sn : p.o2_sn;
                T *orow = base + (int64_t)b * sb + (int64_t)h * sh + (int64_t)row * sn;
                const uint32_t acc_col = o == 0 ? ACC1_COL : ACC2_COL;
#pragma unroll 1
                for (int c = 0; c < D / 64; ++c) {
                    const int col = half * (D / 2) + c * 32;
                    uint32_t r[32];
                    if (nit > 0) {
                        tmem_ld32(lane_base + acc_col + col, r);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = 0u;
                    }
                    if (row < limit) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 v;
                            v.x = pack16b<BF16>(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                            v.y = pack16b<BF16>(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                            v.z = pack16b<BF16>(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                            v.w = pack16b<BF16>(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                            *reinterpret_cast<uint4 *>(orow + col + i) = v;
                        }
                    }
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Host
// ---------------------------------------------------------------------------
bool tmem_bwd_eligible(const AttnParams &p) {
    return (p.d == 64 || p.d == 128) && p.Tq >= 1 && p.Tk >= 1 && p.vec_q && p.vec_k && p.vec_v && p.vec_do &&
           p.vec_dq && p.vec_dk && p.vec_dv;
}

template <int D, bool BF16, bool DKDV>
static int launch_bwd_tmem(const BwdTmaParams &bp, int nblocks, int BH, cudaStream_t st) {
    const size_t smem = sizeof(BwdTmaSmem<D>) + 1024;
    if (int e = cuda_status(cudaFuncSetAttribute(attn_bwd_tmem<D, BF16, DKDV>,
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)))
        return e;
    dim3 grid(nblocks, BH);
    attn_bwd_tmem<D, BF16, DKDV><<<grid, BWD_THREADS, smem, st>>>(bp);
    count_launch();
    return check_launch();
}

template <int D, bool BF16>
static int bwd_both(BwdTmaParams &bp, const AttnParams &p, cudaStream_t st) {
    const int BH = p.B * p.H;
    bp.out1 = p.dv; bp.o1_sb = p.dv_sb; bp.o1_sh = p.dv_sh; bp.o1_sn = p.dv_sn;
    bp.out2 = p.dk; bp.o2_sb = p.dk_sb; bp.o2_sh = p.dk_sh; bp.o2_sn = p.dk_sn;
    if (int e = launch_bwd_tmem<D, BF16, true>(bp, (p.Tk + BT - 1) / BT, BH, st)) return e;
    bp.out1 = p.dq; bp.o1_sb = p.dq_sb; bp.o1_sh = p.dq_sh; bp.o1_sn = p.dq_sn;
    bp.out2 = nullptr;
    return launch_bwd_tmem<D, BF16, false>(bp, (p.Tq + BT - 1) / BT, BH, st);
}

// delta must already be in p.delta (the caller runs the delta kernel first).
int tmem_bwd(const AttnParams &p, int dtype, cudaStream_t st) {
    BwdTmaParams bp{};
    const bool bf16 = dtype == RGD_BF16;
    if (int e = encode_heads_map(&bp.mq, p.q, p.B, p.H, p.Tq, p.d, p.q_sb, p.q_sh, p.q_sn, 64, BT, bf16)) return e;
    if (int e = encode_heads_map(&bp.mk, p.k, p.B, p.H, p.Tk, p.d, p.k_sb, p.k_sh, p.k_sn, 64, BT, bf16)) return e;
    if (int e = encode_heads_map(&bp.mv, p.v, p.B, p.H, p.Tk, p.d, p.v_sb, p.v_sh, p.v_sn, 64, BT, bf16)) return e;
    if (int e = encode_heads_map(&bp.mdo, p.d_o, p.B, p.H, p.Tq, p.d, p.do_sb, p.do_sh, p.do_sn, 64, BT, bf16)) return e;
    bp.bias = p.bias; bp.b_sb = p.b_sb; bp.b_sh = p.b_sh; bp.b_sq = p.b_sq;
    bp.bias_kind = p.bias_kind; bp.bias_f32 = p.bias_f32; bp.bias_vec = 0;
    bp.lse = p.lse; bp.delta = p.delta;
    bp.H = p.H; bp.Tq = p.Tq; bp.Tk = p.Tk; bp.Tq_rounded = p.Tq_rounded; bp.causal = p.causal;
    bp.scale = p.scale; bp.scale_log2 = p.scale * LOG2E;
    bp.status = tmem_status_ptr();
    if (!bp.status) return RGD_E_DEVICE;
    if (p.d == 128) return bf16 ? bwd_both<128, true>(bp, p, st) : bwd_both<128, false>(bp, p, st);
    return bf16 ? bwd_both<64, true>(bp, p, st) : bwd_both<64, false>(bp, p, st);
}

}  // namespace attn
}  // namespace rgd
