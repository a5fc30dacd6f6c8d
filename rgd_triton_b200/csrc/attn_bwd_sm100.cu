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
bool bias_tma_ok(const AttnParams &p);
int encode_bias_map(rgd_cache *cache, CUtensorMap *out, const AttnParams &p, bool bf16, int box_q);

constexpr int BWD_THREADS = 320;
constexpr int DKDV_SUB_THREADS = 384;   // 8 compute warps, TMA producer, three MMA issuers
constexpr int SINGLE64_THREADS = 512;   // the same plus four warps that read dQ partial tiles back
constexpr int BT = 128;   // tile edge (queries and keys)

struct BwdTmaParams {
    CUtensorMap mq, mk, mv, mdo;
    void *out1, *out2;                  // DKDV: dV, dK.  DQ: dQ, unused.
    int64_t o1_sb, o1_sh, o1_sn, o2_sb, o2_sh, o2_sn;
    const void *bias;
    int64_t b_sb, b_sh, b_sq;
    int bias_kind, bias_f32, bias_vec;
    CUtensorMap mbias;                  // BIAS == 2: (Tk, Tq, H or 1, B or 1) map over the bias, box 64 x 128
    CUtensorMap mbias64;                // the same tensor with box 64 keys x 64 queries (dK/dV sub-blocks)
    int bias_h0, bias_b0;               // bias broadcast over heads / batch: coordinate 0
    const float *lse2, *delta_s;        // [B, H, Tq128]: lse * log2(e) (+inf past Tq), delta * scale (0 past Tq)
    int H, Tq, Tk, Tq128, causal;
    float scale, scale_log2;
    int *status;
    // bias gradient (null when not wanted): vector form fp32 [B, H, Tk], matrix form [B, H, Tq, Tk] in
    // the tensor dtype; the kernels hold dS = scale * P (dP - delta), so they multiply by 1 / scale
    void *dbias;
    int64_t db_sb, db_sh, db_sq;
    int dbias_vec;
    float inv_scale;
    // matrix bias with tile lists (optional, never with a causal mask): per key block of each bias
    // slice the query blocks to visit (dK/dV kernel), per query block the key blocks (dQ kernel)
    const uint16_t *tlk_cnt, *tlk_list, *tlq_cnt, *tlq_list;
    int tl_nqb, tl_nkb;
    float *dq_acc;                      // single-pass form (head_dim 64): fp32 dQ accumulator [B, H, 16, Tq128, 4], else null
};

// BSTAGES: stages of TMA-staged bias tiles (query rows x key columns, 16-bit, two
// 64-column panels with 128-byte swizzle); 0 when the bias does not go through TMA.
template <int D, int BSTAGES>
struct alignas(1024) BwdTmaSmem {
    unsigned char x1[BT * D * 2], x2[BT * D * 2];            // fixed tiles
    unsigned char y1[2][BT * D * 2], y2[2][BT * D * 2];      // looped tiles, 2 stages
    unsigned char bias[BSTAGES > 0 ? BSTAGES : 1][BSTAGES > 0 ? BT * BT * 2 : 1024];
    // dK/dV: row statistics of the staged query block (not with head_dim 128 and staged bias
    // tiles: shared memory is full there and the statistics are read from global memory)
    static constexpr int NSTAT = (D == 128 && BSTAGES > 0) ? 4 : BT;
    alignas(16) float lse_s[2][NSTAT], dsc_s[2][NSTAT];
    uint64_t x_full, g1_full, g2_full, p_ready, ds_ready, acc_full;
    uint64_t y_full[2], y_empty[2];
    uint64_t bb_full[2], bb_empty[2];
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

// BIAS: whether an additive bias exists; the no-bias instantiation carries none of
// the bias code (and none of its register pressure).
// (BIAS: 0 none, 1 read from global memory by the compute threads, 2 staged through TMA.)

template <int D, bool BF16, bool DKDV, int BIAS>
__global__ void __launch_bounds__(BWD_THREADS, 1) attn_bwd_tmem(const __grid_constant__ BwdTmaParams p) {
    constexpr int BSTAGES = BIAS == 2 ? (D == 64 ? 2 : 1) : 0;
    constexpr bool STAGE_STATS = DKDV && !(D == 128 && BSTAGES > 0);
    constexpr uint32_t BIAS_BYTES = BT * BT * 2;
    constexpr int HALVES = D / 64;
    constexpr uint32_t PANEL = 128 * 64 * 2;
    constexpr uint32_t TILE_BYTES = BT * D * 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t G1_COL = 0, G2_COL = 128, ACC1_COL = 256, ACC2_COL = 384;
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;

    extern __shared__ unsigned char smem_raw[];
    BwdTmaSmem<D, BSTAGES> &sm = *reinterpret_cast<BwdTmaSmem<D, BSTAGES> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

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
            mbar_init(&sm.bb_full[s], 1);
            mbar_init(&sm.bb_empty[s], 256);
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
            if constexpr (BIAS == 2) tma_prefetch_desc(&p.mbias);
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
                mbar_expect_tx(&sm.y_full[s], 2 * TILE_BYTES + (STAGE_STATS ? 2 * BT * 4 : 0));
                const int row = (i_begin + it) * BT;
                for (int hh = 0; hh < HALVES; ++hh) {
                    tma_load_4d(sm.y1[s] + hh * PANEL, my1, &sm.y_full[s], hh * 64, row, h, b);
                    tma_load_4d(sm.y2[s] + hh * PANEL, my2, &sm.y_full[s], hh * 64, row, h, b);
                }
                if constexpr (STAGE_STATS) {
                    // the query block's lse / delta rows, read by every compute thread in both phases
                    bulk_load_1d(sm.lse_s[s], p.lse2 + (int64_t)bh * p.Tq128 + row, BT * 4, &sm.y_full[s]);
                    bulk_load_1d(sm.dsc_s[s], p.delta_s + (int64_t)bh * p.Tq128 + row, BT * 4, &sm.y_full[s]);
                }
                if constexpr (BIAS == 2) {
                    const int sb = it % BSTAGES;
                    ok = mbar_wait(&sm.bb_empty[sb], ((uint32_t)(it / BSTAGES) & 1u) ^ 1u, status, 42);
                    if (!ok) break;
                    mbar_expect_tx(&sm.bb_full[sb], BIAS_BYTES);
                    // tile rows are queries, columns keys
                    const int qrow = DKDV ? row : r0, kcol = DKDV ? r0 : row;
                    for (int pn = 0; pn < 2; ++pn)
                        tma_load_4d(sm.bias[sb] + pn * (BT * 128), &p.mbias, &sm.bb_full[sb], kcol + pn * 64, qrow,
                                    p.bias_h0 ? 0 : h, p.bias_b0 ? 0 : b);
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
        const float *lse2_bh = p.lse2 + (int64_t)bh * p.Tq128;
        const float *ds_bh = p.delta_s + (int64_t)bh * p.Tq128;
        const char *bias_bh = nullptr;
        if constexpr (BIAS == 1)
            bias_bh = reinterpret_cast<const char *>(p.bias) +
                      ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : 2);

        // DQ: per-thread row statistics (rows past Tq hold +inf / 0, so they yield P = 0)
        float lse_row = INFINITY, dsc_row = 0.f;
        if (!DKDV) {
            lse_row = lse2_bh[row];
            dsc_row = ds_bh[row];
        }
        const bool cta_key_tail = DKDV && (r0 + BT > p.Tk);

        bool ok = true;
        for (int it = 0; it < nit; ++it) {
            const uint32_t par = (uint32_t)it & 1u;
            const int blk0 = (i_begin + it) * BT;          // first column index of this block
            const int c0 = blk0 + half * 64;               // first column this thread handles
            // Blocks that need per-element masking: the diagonal block under the causal
            // mask, and any block touching the end of the keys.  Rows / columns past
            // the end of the QUERIES need nothing: their lse2 is +inf.
            const bool diag = p.causal && (DKDV ? (blk0 == r0) : (blk0 + BT > r0));
            const bool slow = BIAS != 0 || diag || cta_key_tail || (!DKDV && blk0 + BT > p.Tk);
            float pv[64];

            // Bias for this thread's 64 elements, fetched before waiting for the score tile so
            // the loads overlap the wait.  Indices are clamped to stay in bounds; elements
            // past the ends are masked below.
            float bv[BIAS != 0 ? 64 : 1];
            if constexpr (BIAS == 2) {
                const int sb = it % BSTAGES;
                ok = mbar_wait(&sm.bb_full[sb], (uint32_t)(it / BSTAGES) & 1u, status, 65);
                if (!ok) break;
                const unsigned char *tile = sm.bias[sb];
                if (DKDV) {
                    // thread = key column row_l of the tile, 64 query rows half*64 .. +63
                    const unsigned char *colp = tile + (row_l >> 6) * (BT * 128) + (row_l & 7) * 2;
                    const int kc = (row_l & 63) >> 3;
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const int qr = half * 64 + i;
                        bv[i] = to_f32<T>(*reinterpret_cast<const T *>(colp + qr * 128 + ((kc ^ (qr & 7)) << 4)));
                    }
                } else {
                    // thread = query row row_l, 64 key columns = the whole 128-byte row of panel `half`
                    const unsigned char *rowp = tile + half * (BT * 128) + row_l * 128;
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        union { uint4 u; T v[8]; } cv;
                        cv.u = *reinterpret_cast<const uint4 *>(rowp + ((c ^ (row_l & 7)) << 4));
#pragma unroll
                        for (int e = 0; e < 8; ++e) bv[8 * c + e] = to_f32<T>(cv.v[e]);
                    }
                }
                // (the stage is handed back at the end of the iteration, once instructions that
                // consume these values have been issued: an arrive right here could be performed
                // while the loads above are still in flight, and with a single stage the refill
                // by the copy engine follows at once)
            }
            if constexpr (BIAS == 1) {
                if (DKDV) {
                    const int kj = min(row, p.Tk - 1);
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const int qi = min(c0 + i, p.Tq - 1);
                        const int64_t off = (p.bias_kind == RGD_BIAS_MATRIX ? (int64_t)qi * p.b_sq : 0) + kj;
                        bv[i] = p.bias_f32 ? __ldg(reinterpret_cast<const float *>(bias_bh) + off)
                                           : to_f32<T>(reinterpret_cast<const T *>(bias_bh)[off]);
                    }
                } else {
                    const int qi = min(row, p.Tq - 1);
                    const int64_t off = (p.bias_kind == RGD_BIAS_MATRIX ? (int64_t)qi * p.b_sq : 0) + c0;
                    if (!p.bias_f32 && p.bias_vec && c0 + 64 <= p.Tk) {
                        const T *src = reinterpret_cast<const T *>(bias_bh) + off;
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const Vec<T, 8> v = load_vec<T, 8>(src + 8 * i);
#pragma unroll
                            for (int e = 0; e < 8; ++e) bv[8 * i + e] = to_f32<T>(v.v[e]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 64; ++i) {
                            const int64_t o2 = off + min(i, p.Tk - 1 - c0 < 0 ? 0 : p.Tk - 1 - c0);
                            bv[i] = p.bias_f32 ? __ldg(reinterpret_cast<const float *>(bias_bh) + o2)
                                               : to_f32<T>(reinterpret_cast<const T *>(bias_bh)[o2]);
                        }
                    }
                }
            }
            // row statistics of this query block: staged in shared memory, else straight from global
            const float *lse_blk = STAGE_STATS ? sm.lse_s[it & 1] : lse2_bh + blk0;
            const float *dsc_blk = STAGE_STATS ? sm.dsc_s[it & 1] : ds_bh + blk0;
            if (STAGE_STATS) {
                ok = mbar_wait(&sm.y_full[it & 1], (uint32_t)(it >> 1) & 1u, status, 60);
                if (!ok) break;
            }
            ok = mbar_wait(&sm.g1_full, par, status, 61);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t ra[32], rb[32];
                tmem_ld32(lane_base + G1_COL + half * 64, ra);
                tmem_ld32(lane_base + G1_COL + half * 64 + 32, rb);
                if (!DKDV) {
                    // dQ: P stays in registers, so the score columns are free as soon as they
                    // have been read and the next block's score GEMM runs under the exponentials
                    tmem_wait_ld();
                    tc_fence_before_sync();
                    mbar_arrive(&sm.p_ready);
                }
                if (!slow) {
                    if (DKDV) {
                        float4 l4[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) l4[i] = reinterpret_cast<const float4 *>(lse_blk + half * 64)[i];
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            pv[4 * i + 0] = ex2b(fmaf(__uint_as_float(ra[4 * i + 0]), p.scale_log2, -l4[i].x));
                            pv[4 * i + 1] = ex2b(fmaf(__uint_as_float(ra[4 * i + 1]), p.scale_log2, -l4[i].y));
                            pv[4 * i + 2] = ex2b(fmaf(__uint_as_float(ra[4 * i + 2]), p.scale_log2, -l4[i].z));
                            pv[4 * i + 3] = ex2b(fmaf(__uint_as_float(ra[4 * i + 3]), p.scale_log2, -l4[i].w));
                            pv[32 + 4 * i + 0] = ex2b(fmaf(__uint_as_float(rb[4 * i + 0]), p.scale_log2, -l4[8 + i].x));
                            pv[32 + 4 * i + 1] = ex2b(fmaf(__uint_as_float(rb[4 * i + 1]), p.scale_log2, -l4[8 + i].y));
                            pv[32 + 4 * i + 2] = ex2b(fmaf(__uint_as_float(rb[4 * i + 2]), p.scale_log2, -l4[8 + i].z));
                            pv[32 + 4 * i + 3] = ex2b(fmaf(__uint_as_float(rb[4 * i + 3]), p.scale_log2, -l4[8 + i].w));
                        }
                    } else {
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            pv[i] = ex2b(fmaf(__uint_as_float(ra[i]), p.scale_log2, -lse_row));
                            pv[32 + i] = ex2b(fmaf(__uint_as_float(rb[i]), p.scale_log2, -lse_row));
                        }
                    }
                } else {
                    tmem_wait_ld();
                    // Interior blocks with a bias need no mask either: rows past the end of Q have
                    // lse2 = +inf, which makes their P exactly 0 whatever the (clamped) bias holds.
                    const bool need_mask = diag || cta_key_tail || (!DKDV && blk0 + BT > p.Tk);
                    if (!need_mask) {
#pragma unroll
                        for (int i = 0; i < 64; ++i) {
                            float x = __uint_as_float(i < 32 ? ra[i & 31] : rb[i & 31]) * p.scale_log2;
                            const float l2 = DKDV ? lse_blk[half * 64 + i] : lse_row;
                            if constexpr (BIAS != 0) x = fmaf(bv[i], LOG2E, x);
                            pv[i] = ex2b(x - l2);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 64; ++i) {
                            const int col = c0 + i;
                            const int qi = DKDV ? col : row, kj = DKDV ? row : col;
                            float x = __uint_as_float(i < 32 ? ra[i & 31] : rb[i & 31]) * p.scale_log2;
                            const bool masked = kj >= p.Tk || qi >= p.Tq || (p.causal && kj > qi);
                            const float l2 = DKDV ? lse_blk[half * 64 + i] : lse_row;
                            if constexpr (BIAS != 0) x = fmaf(bv[i], LOG2E, x);
                            pv[i] = masked ? 0.f : ex2b(x - l2);
                        }
                    }
                }
                if (DKDV) {
                    uint32_t pk[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) pk[i] = pack16b<BF16>(pv[2 * i], pv[2 * i + 1]);
                    tmem_st32(lane_base + G1_COL + half * 64, pk);
                    tmem_wait_st();
                    tc_fence_before_sync();
                    mbar_arrive(&sm.p_ready);
                }
            }
            ok = mbar_wait(&sm.g2_full, par, status, 62);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t ga[32], gb[32];
                tmem_ld32(lane_base + G2_COL + half * 64, ga);
                tmem_ld32(lane_base + G2_COL + half * 64 + 32, gb);
                uint32_t pk[32];
                if (DKDV) {
                    float4 d4[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) d4[i] = reinterpret_cast<const float4 *>(dsc_blk + half * 64)[i];
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float a0 = pv[4 * i + 0] * fmaf(__uint_as_float(ga[4 * i + 0]), p.scale, -d4[i].x);
                        const float a1 = pv[4 * i + 1] * fmaf(__uint_as_float(ga[4 * i + 1]), p.scale, -d4[i].y);
                        const float a2 = pv[4 * i + 2] * fmaf(__uint_as_float(ga[4 * i + 2]), p.scale, -d4[i].z);
                        const float a3 = pv[4 * i + 3] * fmaf(__uint_as_float(ga[4 * i + 3]), p.scale, -d4[i].w);
                        pk[2 * i] = pack16b<BF16>(a0, a1);
                        pk[2 * i + 1] = pack16b<BF16>(a2, a3);
                        const float b0 = pv[32 + 4 * i + 0] * fmaf(__uint_as_float(gb[4 * i + 0]), p.scale, -d4[8 + i].x);
                        const float b1 = pv[32 + 4 * i + 1] * fmaf(__uint_as_float(gb[4 * i + 1]), p.scale, -d4[8 + i].y);
                        const float b2 = pv[32 + 4 * i + 2] * fmaf(__uint_as_float(gb[4 * i + 2]), p.scale, -d4[8 + i].z);
                        const float b3 = pv[32 + 4 * i + 3] * fmaf(__uint_as_float(gb[4 * i + 3]), p.scale, -d4[8 + i].w);
                        pk[16 + 2 * i] = pack16b<BF16>(b0, b1);
                        pk[16 + 2 * i + 1] = pack16b<BF16>(b2, b3);
                    }
                } else {
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float a0 = pv[2 * i] * fmaf(__uint_as_float(ga[2 * i]), p.scale, -dsc_row);
                        const float a1 = pv[2 * i + 1] * fmaf(__uint_as_float(ga[2 * i + 1]), p.scale, -dsc_row);
                        pk[i] = pack16b<BF16>(a0, a1);
                        const float b0 = pv[32 + 2 * i] * fmaf(__uint_as_float(gb[2 * i]), p.scale, -dsc_row);
                        const float b1 = pv[32 + 2 * i + 1] * fmaf(__uint_as_float(gb[2 * i + 1]), p.scale, -dsc_row);
                        pk[16 + i] = pack16b<BF16>(b0, b1);
                    }
                }
                tmem_st32(lane_base + G2_COL + half * 64, pk);
                tmem_wait_st();
            }
            tc_fence_before_sync();
            mbar_arrive(&sm.ds_ready);
            // dS, which depends on every bias value read above, has been stored: the bias stage is free
            if constexpr (BIAS == 2) mbar_arrive(&sm.bb_empty[it % BSTAGES]);
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
// dK / dV without bias, sub-block pipelined.  Same roles and tiles as MODE 1 above,
// but each 128-query block is processed as two 64-query sub-blocks whose score
// columns are double-buffered in tensor memory: G1 / P of sub-block parity b in
// columns [b*64, b*64+64), G2 / dS in [128 + b*64, ...).  While the compute warps
// turn sub-block u's scores into P and dS, the tensor cores run the accumulation
// GEMMs of sub-block u-1 and the score GEMMs of sub-block u+1, so the exponentials
// leave the critical path (at the price of N = 64 score GEMMs).
// ---------------------------------------------------------------------------
// BIAS: a matrix bias in the tensor dtype, staged by TMA as one 64-query x 128-key sub-tile per
// sub-block (two 64-key panels, 128-byte swizzle); stage b belongs to the compute group that
// owns sub-blocks of parity b, which frees it for the next block as soon as its P is formed.
// With head_dim 128 and a bias the row statistics are not staged (shared memory is full):
// they are read from global memory, where every warp reads the same cached words.
template <int D, bool BIAS>
struct alignas(1024) DkdvSubSmem {
    static constexpr bool STAGE_STATS = !(BIAS && D == 128);
    unsigned char x1[BT * D * 2], x2[BT * D * 2];            // K, V
    unsigned char y1[2][BT * D * 2], y2[2][BT * D * 2];      // Q, dO, 2 stages
    unsigned char bias[BIAS ? 2 : 1][BIAS ? 64 * BT * 2 : 1024];
    alignas(16) float lse_s[2][STAGE_STATS ? BT : 4], dsc_s[2][STAGE_STATS ? BT : 4];   // row statistics of the staged query block
    uint64_t x_full, acc_full;
    uint64_t y_full[2], y_empty[2];
    uint64_t g1_full[2], g2_full[2], p_ready[2], ds_ready[2];   // per sub-block parity
    uint64_t g1_free[2], g2_free[2];                            // accumulation GEMM has read P / dS
    uint64_t bb_full[2], bb_empty[2];                           // bias sub-tile of parity b
    int qblk[2];                                                // query block index of the staged block (tile lists)
    uint32_t tmem_base;
};

// BIASM: 0 no bias, 1 matrix bias staged by TMA, 2 vector bias (one value per key = per thread),
// 3 matrix bias with tile lists (an instantiation of its own: the list plumbing costs the dense
// form 5-11 % when it shares the code).
template <int D, bool BF16, int BIASM>
__global__ void __launch_bounds__(DKDV_SUB_THREADS, 1) attn_bwd_dkdv_sub(const __grid_constant__ BwdTmaParams p) {
    constexpr bool BIAS = BIASM == 1 || BIASM == 3;
    constexpr bool LISTS = BIASM == 3;
    using Smem = DkdvSubSmem<D, BIAS>;
    constexpr bool STAGE_STATS = Smem::STAGE_STATS;
    constexpr uint32_t BIAS_BYTES = 64 * BT * 2;
    constexpr int HALVES = D / 64;
    constexpr uint32_t PANEL = 128 * 64 * 2;
    constexpr uint32_t TILE_BYTES = BT * D * 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t G1_COL = 0, G2_COL = 128, ACC1_COL = 256, ACC2_COL = 384;
    constexpr uint32_t SUB_ROWS = 64 * 128;          // byte offset of query row 64 inside a panel
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;

    extern __shared__ unsigned char smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int r0 = blk * BT;                               // first key of this CTA
    const int i_begin = p.causal ? r0 / BT : 0;
    const int i_end = (p.Tq + BT - 1) / BT;
    // With tile lists (matrix bias only) the CTA visits the listed query blocks: the count bounds
    // every role's loop, the TMA producer alone reads the list and posts each stage's block index
    // in shared memory (sm.qblk) before the stage's barrier, where the compute threads pick it up.
    int tl_idx = -1;
    if constexpr (LISTS)
        tl_idx = (int)(((p.bias_b0 ? 0 : b) * (p.bias_h0 ? 1 : p.H) + (p.bias_h0 ? 0 : h)) * (int)gridDim.x + blk);
    const int nit = LISTS ? (int)p.tlk_cnt[LISTS ? tl_idx : 0] : max(i_end - i_begin, 0);
    const int nsub = 2 * nit;
    int *status = p.status;

    if (threadIdx.x == 0) {
        mbar_init(&sm.x_full, 1);
        mbar_init(&sm.acc_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.y_full[s], 1);
            mbar_init(&sm.y_empty[s], 1);
            mbar_init(&sm.g1_full[s], 1);
            mbar_init(&sm.g2_full[s], 1);
            mbar_init(&sm.g1_free[s], 1);
            mbar_init(&sm.g2_free[s], 1);
            mbar_init(&sm.p_ready[s], 128);
            mbar_init(&sm.ds_ready[s], 128);
            mbar_init(&sm.bb_full[s], 1);
            mbar_init(&sm.bb_empty[s], 128);
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
            tma_prefetch_desc(&p.mk);
            tma_prefetch_desc(&p.mv);
            tma_prefetch_desc(&p.mq);
            tma_prefetch_desc(&p.mdo);
            if constexpr (BIAS) tma_prefetch_desc(&p.mbias64);
            mbar_expect_tx(&sm.x_full, 2 * TILE_BYTES);
            for (int hh = 0; hh < HALVES; ++hh) {
                tma_load_4d(sm.x1 + hh * PANEL, &p.mk, &sm.x_full, hh * 64, r0, h, b);
                tma_load_4d(sm.x2 + hh * PANEL, &p.mv, &sm.x_full, hh * 64, r0, h, b);
            }
            bool ok = true;
            // the list entry of the next block is fetched while waiting for this block's stage
            const uint16_t *lst = LISTS ? p.tlk_list + (int64_t)tl_idx * p.tl_nqb : nullptr;
            int qb_next = LISTS ? (int)lst[0] : 0;
            for (int it = 0; it < nit; ++it) {
                const int s = it & 1;
                const uint32_t ph = (uint32_t)(it >> 1) & 1u;
                int qb = i_begin + it;
                if constexpr (LISTS) {
                    qb = qb_next;
                    if (it + 1 < nit) qb_next = lst[it + 1];
                }
                ok = mbar_wait(&sm.y_empty[s], ph ^ 1u, status, 71);
                if (!ok) break;
                if constexpr (LISTS) sm.qblk[s] = qb;   // ordered before the arrive below (release), read after the wait on y_full
                mbar_expect_tx(&sm.y_full[s], 2 * TILE_BYTES + (STAGE_STATS ? 2 * BT * 4 : 0));
                const int row = qb * BT;
                if constexpr (STAGE_STATS) {
                    bulk_load_1d(sm.lse_s[s], p.lse2 + (int64_t)bh * p.Tq128 + row, BT * 4, &sm.y_full[s]);
                    bulk_load_1d(sm.dsc_s[s], p.delta_s + (int64_t)bh * p.Tq128 + row, BT * 4, &sm.y_full[s]);
                }
                for (int hh = 0; hh < HALVES; ++hh) {
                    tma_load_4d(sm.y1[s] + hh * PANEL, &p.mq, &sm.y_full[s], hh * 64, row, h, b);
                    tma_load_4d(sm.y2[s] + hh * PANEL, &p.mdo, &sm.y_full[s], hh * 64, row, h, b);
                }
                if constexpr (BIAS) {
                    // sub-tile of sub-block parity sb: queries row + 64 sb .. + 63, keys r0 .. r0 + 127
                    for (int sb = 0; sb < 2 && ok; ++sb) {
                        ok = mbar_wait(&sm.bb_empty[sb], ((uint32_t)it & 1u) ^ 1u, status, 72);
                        if (!ok) break;
                        mbar_expect_tx(&sm.bb_full[sb], BIAS_BYTES);
                        for (int pn = 0; pn < 2; ++pn)
                            tma_load_4d(sm.bias[sb] + pn * (64 * 128), &p.mbias64, &sm.bb_full[sb], r0 + pn * 64,
                                        row + sb * 64, p.bias_h0 ? 0 : h, p.bias_b0 ? 0 : b);
                    }
                    if (!ok) break;
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 9 || warp == 10) {
        // ------------- MMA issuers A1 / A2: the score GEMMs K Q^T and V dO^T -------------
        // One thread can issue an MMA only every ~54 clocks whatever its size, which is as long
        // as these N = 64 MMAs take to run, so each kind of GEMM gets its own issuing thread.
        if (lane == 0 && nit > 0) {
            const bool second = warp == 10;
            constexpr uint32_t idesc_g = make_idesc(BF16, BT, 64, false, false);
            // Descriptors of the operand tiles, encoded once; the loop below only adds offsets.
            const uint64_t dx = make_sdesc(smem_u32(second ? sm.x2 : sm.x1), 16, 1024);
            uint64_t dyk[2];                                 // Q (or dO) per stage, K-major view
#pragma unroll
            for (int s = 0; s < 2; ++s) dyk[s] = make_sdesc(smem_u32(second ? sm.y2[s] : sm.y1[s]), 16, 1024);
            const uint32_t gcol = tbase + (second ? G2_COL : G1_COL);
            uint64_t *full = second ? sm.g2_full : sm.g1_full, *free_ = second ? sm.g2_free : sm.g1_free;
            bool ok = mbar_wait(&sm.x_full, 0, status, 81);
            for (int u = 0; u < nsub && ok; ++u) {
                const int sb = u & 1, it = u >> 1, s = it & 1;
                if (sb == 0) {
                    ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 82);
                    if (!ok) break;
                }
                // the columns are free once the accumulation GEMM of sub-block u - 2 has read them
                if (u >= 2) {
                    ok = mbar_wait(&free_[sb], (uint32_t)(it - 1) & 1u, status, 85);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                // [128 keys] x [64 queries of sub-block u], contraction over channels
                const uint64_t ydu = sdesc_advance(dyk[s], sb * SUB_ROWS);
                const uint32_t dcol = gcol + sb * 64;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * PANEL + (kk % 4) * 32;
                    umma_ss(dcol, sdesc_advance(dx, off), sdesc_advance(ydu, off), idesc_g, kk > 0);
                }
                umma_commit(&full[sb]);
            }
        }
    } else if (warp == 11) {
        // ------------------- MMA issuer B: the accumulation GEMMs -------------------
        // All MMAs that add into dV / dK come from this one thread, in sub-block order, so the
        // order of the floating-point sums is fixed.
        if (lane == 0 && nit > 0) {
            constexpr uint32_t idesc_acc = make_idesc(BF16, BT, D, false, true);
            uint64_t dy1m[2], dy2m[2];                       // Q / dO per stage, MN-major view
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                dy1m[s] = make_sdesc(smem_u32(sm.y1[s]), PANEL, 1024);
                dy2m[s] = make_sdesc(smem_u32(sm.y2[s]), PANEL, 1024);
            }
            // accumulation GEMM of sub-block u: contraction over its 64 queries (4 steps of 16),
            // packed two per column into the first 32 columns of the sub-block's score columns
            auto issue_acc = [&](int u, uint32_t acc_col, uint32_t a_col, uint64_t yd) {
                const uint64_t ydu = sdesc_advance(yd, (u & 1) * SUB_ROWS);
                const uint32_t acol = tbase + a_col + (u & 1) * 64;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_ts(tbase + acc_col, acol + kk * 8, sdesc_advance(ydu, kk * 2048), idesc_acc, u > 0 || kk > 0);
            };
            bool ok = true;
            for (int u = 0; u < nsub && ok; ++u) {
                const int sb = u & 1, it = u >> 1, s = it & 1;
                const uint32_t par = (uint32_t)it & 1u;
                if (sb == 0) {
                    ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 87);
                    if (!ok) break;
                }
                ok = mbar_wait(&sm.p_ready[sb], par, status, 83);
                if (!ok) break;
                tc_fence_after_sync();
                issue_acc(u, ACC1_COL, G1_COL, dy2m[s]);            // dV += P^T dO
                tc_fence_before_sync();
                mbar_arrive(&sm.g1_free[sb]);   // issued, not finished: the tensor pipe runs MMAs in issue order
                ok = mbar_wait(&sm.ds_ready[sb], par, status, 84);
                if (!ok) break;
                tc_fence_after_sync();
                issue_acc(u, ACC2_COL, G2_COL, dy1m[s]);            // dK += dS^T Q
                tc_fence_before_sync();
                mbar_arrive(&sm.g2_free[sb]);
                if (sb == 1) umma_commit(&sm.y_empty[s]);            // both sub-blocks of this block consumed
            }
            umma_commit(&sm.acc_full);
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        // Warps 0-3 own the even sub-blocks, warps 4-7 the odd ones: each thread handles one
        // key row and all 64 queries of its sub-block, and the two groups run half a period
        // apart, so one group's exponentials overlap the other's tensor-memory round trips.
        const int row_l = (warp & 3) * 32 + lane;          // key row of the tile == TMEM lane
        const int sb = warp >> 2;                          // sub-block parity this warp group owns
        const int half = sb;                               // epilogue: which half of the channels
        const int row = r0 + row_l;
        const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        const bool cta_key_tail = r0 + BT > p.Tk;
        const uint32_t col = sb * 64;                      // this group's columns inside G1 / G2
        // vector bias: this thread's key has one value for every query, times log2(e)
        float bk2 = 0.f;
        if constexpr (BIASM == 2) {
            if (row < p.Tk) {
                const char *bias_bh = reinterpret_cast<const char *>(p.bias) +
                                      ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : 2);
                bk2 = (p.bias_f32 ? reinterpret_cast<const float *>(bias_bh)[row]
                                  : to_f32<T>(reinterpret_cast<const T *>(bias_bh)[row])) * LOG2E;
            }
        }

        float bsum = 0.f;                                  // vector-bias gradient of this key over this group's queries
        bool ok = true;
        for (int it = 0; it < nit; ++it) {
            const uint32_t par = (uint32_t)it & 1u;
            const int s = it & 1;
            int blk0 = (i_begin + it) * BT;
            if constexpr (LISTS) {
                // the block's index is posted with its tiles
                ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 90);
                if (!ok) break;
                blk0 = sm.qblk[s] * BT;
            }
            const int c0 = blk0 + sb * 64;                 // first query of the sub-block
            const bool slow = cta_key_tail || (p.causal && blk0 == r0);
            // row statistics of this sub-block's 64 queries: staged in shared memory, else from global
            const float *lse_f = STAGE_STATS ? &sm.lse_s[s][sb * 64] : p.lse2 + (int64_t)bh * p.Tq128 + c0;
            const float *dsc_f = STAGE_STATS ? &sm.dsc_s[s][sb * 64] : p.delta_s + (int64_t)bh * p.Tq128 + c0;
            const float4 *lse4 = reinterpret_cast<const float4 *>(lse_f);
            const float4 *dsc4 = reinterpret_cast<const float4 *>(dsc_f);
            float pv[64];

            if constexpr (!LISTS) {
                // row statistics of this block have landed
                ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 90);
                if (!ok) break;
            }

            // x0[i] = bias * log2(e) - lse * log2(e) of query i (only -lse without a bias), formed
            // before the scores are waited for
            float x0[BIAS ? 64 : 1];
            if constexpr (BIAS) {
                ok = mbar_wait(&sm.bb_full[sb], (uint32_t)it & 1u, status, 94);
                if (!ok) break;
                // this thread's key column of the sub-tile: panel = key / 64, 16-byte chunk index
                // XOR (query mod 8) inside the 128-byte row of query i
                const unsigned char *colp = sm.bias[sb] + (row_l >> 6) * (64 * 128) + (row_l & 7) * 2;
                const int kc = (row_l & 63) >> 3;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 l = lse4[i];
                    const float lv[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int qi = 4 * i + e;
                        const float bvl = to_f32<T>(*reinterpret_cast<const T *>(colp + qi * 128 + ((kc ^ (qi & 7)) << 4)));
                        x0[qi] = fmaf(bvl, LOG2E, -lv[e]);
                    }
                }
            }
            ok = mbar_wait(&sm.g1_full[sb], par, status, 91);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t ra[32], rb[32];
                tmem_ld32(lane_base + G1_COL + col, ra);
                tmem_ld32(lane_base + G1_COL + col + 32, rb);
                tmem_wait_ld();
                if (!slow) {
                    if constexpr (BIAS) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            pv[i] = ex2b(fmaf(__uint_as_float(ra[i]), p.scale_log2, x0[i]));
                            pv[32 + i] = ex2b(fmaf(__uint_as_float(rb[i]), p.scale_log2, x0[32 + i]));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 l = lse4[i];
                            pv[4 * i + 0] = ex2b(fmaf(__uint_as_float(ra[4 * i + 0]), p.scale_log2, bk2 - l.x));
                            pv[4 * i + 1] = ex2b(fmaf(__uint_as_float(ra[4 * i + 1]), p.scale_log2, bk2 - l.y));
                            pv[4 * i + 2] = ex2b(fmaf(__uint_as_float(ra[4 * i + 2]), p.scale_log2, bk2 - l.z));
                            pv[4 * i + 3] = ex2b(fmaf(__uint_as_float(ra[4 * i + 3]), p.scale_log2, bk2 - l.w));
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 l = lse4[8 + i];
                            pv[32 + 4 * i + 0] = ex2b(fmaf(__uint_as_float(rb[4 * i + 0]), p.scale_log2, bk2 - l.x));
                            pv[32 + 4 * i + 1] = ex2b(fmaf(__uint_as_float(rb[4 * i + 1]), p.scale_log2, bk2 - l.y));
                            pv[32 + 4 * i + 2] = ex2b(fmaf(__uint_as_float(rb[4 * i + 2]), p.scale_log2, bk2 - l.z));
                            pv[32 + 4 * i + 3] = ex2b(fmaf(__uint_as_float(rb[4 * i + 3]), p.scale_log2, bk2 - l.w));
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const int qi = c0 + i;
                        const bool masked = row >= p.Tk || qi >= p.Tq || (p.causal && row > qi);
                        const float sv = __uint_as_float(i < 32 ? ra[i & 31] : rb[i & 31]);
                        const float off = BIAS ? x0[BIAS ? i : 0] : bk2 - lse_f[i];
                        pv[i] = masked ? 0.f : ex2b(fmaf(sv, p.scale_log2, off));
                    }
                }
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) pk[i] = pack16b<BF16>(pv[2 * i], pv[2 * i + 1]);
                tmem_st32(lane_base + G1_COL + col, pk);
                tmem_wait_st();
            }
            // P, which depends on every bias value read above, is stored: the bias stage is free
            if constexpr (BIAS) mbar_arrive(&sm.bb_empty[sb]);
            tc_fence_before_sync();
            mbar_arrive(&sm.p_ready[sb]);

            ok = mbar_wait(&sm.g2_full[sb], par, status, 92);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t ga[32], gb[32];
                tmem_ld32(lane_base + G2_COL + col, ga);
                tmem_ld32(lane_base + G2_COL + col + 32, gb);
                tmem_wait_ld();
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 dd = dsc4[i];
                    const uint32_t *g = i < 8 ? ga : gb;
                    const int j = (i & 7) * 4;
                    const float a0 = pv[4 * i + 0] * fmaf(__uint_as_float(g[j + 0]), p.scale, -dd.x);
                    const float a1 = pv[4 * i + 1] * fmaf(__uint_as_float(g[j + 1]), p.scale, -dd.y);
                    const float a2 = pv[4 * i + 2] * fmaf(__uint_as_float(g[j + 2]), p.scale, -dd.z);
                    const float a3 = pv[4 * i + 3] * fmaf(__uint_as_float(g[j + 3]), p.scale, -dd.w);
                    pk[2 * i] = pack16b<BF16>(a0, a1);
                    pk[2 * i + 1] = pack16b<BF16>(a2, a3);
                    if constexpr (BIASM == 2) bsum += (a0 + a1) + (a2 + a3);
                }
                tmem_st32(lane_base + G2_COL + col, pk);
                tmem_wait_st();
            }
            tc_fence_before_sync();
            mbar_arrive(&sm.ds_ready[sb]);
        }

        // vector-bias gradient: the two groups each add their half of the queries (two addends:
        // the result does not depend on which lands first)
        if constexpr (BIASM == 2) {
            if (ok && p.dbias != nullptr && row < p.Tk)
                atomicAdd(reinterpret_cast<float *>(p.dbias) + (int64_t)b * p.db_sb + (int64_t)h * p.db_sh + row,
                          bsum * p.inv_scale);
        }
        // epilogue: dV, dK -> global
        if (ok && nit > 0) ok = mbar_wait(&sm.acc_full, 0, status, 93);
        tc_fence_after_sync();
        if (ok) {
#pragma unroll
            for (int o = 0; o < 2; ++o) {
                T *base = reinterpret_cast<T *>(o == 0 ? p.out1 : p.out2);
                const int64_t sb_ = o == 0 ? p.o1_sb : p.o2_sb, sh = o == 0 ? p.o1_sh : p.o2_sh,
                              sn = o == 0 ? p.o1_sn : p.o2_sn;
                T *orow = base + (int64_t)b * sb_ + (int64_t)h * sh + (int64_t)row * sn;
                const uint32_t acc_col = o == 0 ? ACC1_COL : ACC2_COL;
#pragma unroll 1
                for (int c = 0; c < D / 64; ++c) {
                    const int cc = half * (D / 2) + c * 32;
                    uint32_t r[32];
                    if (nit > 0) {
                        tmem_ld32(lane_base + acc_col + cc, r);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = 0u;
                    }
                    if (row < p.Tk) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 v;
                            v.x = pack16b<BF16>(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                            v.y = pack16b<BF16>(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                            v.z = pack16b<BF16>(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                            v.w = pack16b<BF16>(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                            *reinterpret_cast<uint4 *>(orow + cc + i) = v;
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
// Single-pass backward for head_dim 64: the dK/dV kernel above (same roles, tiles, tensor-memory
// map and arithmetic: dK and dV are bit-identical to it) which ALSO forms the dQ partial tile of
// every 128-query block, dQp = dS K, as a fifth GEMM from the dS^T it already holds, and adds it
// to an fp32 accumulator in global memory with 16-byte vector reductions.  No second kernel
// re-reads K, V (and the bias) or recomputes S, dP and the exponentials; a small kernel rounds
// the accumulator into dQ afterwards.  As in the reference (tl.atomic_add into dq,
// flash_attn_triton_cached.py:556-561) the order of the sums into dQ is not fixed: dQ may differ in
// its last bits from run to run, dK and dV do not.  head_dim 64 leaves the 64 tensor-memory
// columns the partial tile needs (448..511) and the shared memory for dS^T (32 KB); at head_dim
// 128 the same scheme is bound by the L2's reduction throughput and loses to the two-kernel form.
// Four extra warps read the partial tiles back, so that reduction stalls do not hold up the
// compute warps; registers are moved between the roles with setmaxnreg.
// ---------------------------------------------------------------------------
template <bool BIAS>
struct alignas(1024) Single64Smem {
    static constexpr int D = 64;
    static constexpr bool STAGE_STATS = true;
    unsigned char x1[BT * D * 2], x2[BT * D * 2];            // K, V
    unsigned char y1[2][BT * D * 2], y2[2][BT * D * 2];      // Q, dO, 2 stages
    unsigned char bias[BIAS ? 2 : 1][BIAS ? 64 * BT * 2 : 1024];
    unsigned char dsm[2 * BT * 64 * 2];                      // dS^T of the block: per sub-block [key][64 queries]
    alignas(16) float lse_s[2][BT], dsc_s[2][BT];            // row statistics of the staged query block
    uint64_t x_full, acc_full;
    uint64_t y_full[2], y_empty[2];
    uint64_t g1_full[2], g2_full[2], p_ready[2], ds_ready[2];
    uint64_t g1_free[2], g2_free[2];
    uint64_t bb_full[2], bb_empty[2];
    uint64_t dq_full, dq_read;                               // dQ partial tile complete / read back
    int qblk[2];
    uint32_t tmem_base;
};

// BIASM: 0 no bias, 1 matrix bias staged by TMA, 2 vector bias.
template <bool BF16, int BIASM>
__global__ void __launch_bounds__(SINGLE64_THREADS, 1) attn_bwd_single64(const __grid_constant__ BwdTmaParams p) {
    static_assert(BIASM >= 0 && BIASM <= 2, "no tile lists here");
    constexpr int D = 64;
    constexpr bool BIAS = BIASM == 1;
    constexpr bool LISTS = false;
    using Smem = Single64Smem<BIAS>;
    constexpr bool STAGE_STATS = Smem::STAGE_STATS;
    constexpr uint32_t BIAS_BYTES = 64 * BT * 2;
    constexpr int HALVES = D / 64;
    constexpr uint32_t PANEL = 128 * 64 * 2;
    constexpr uint32_t TILE_BYTES = BT * D * 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t G1_COL = 0, G2_COL = 128, ACC1_COL = 256, ACC2_COL = 384, DQ_COL = 448;
    constexpr uint32_t SUB_ROWS = 64 * 128;          // byte offset of query row 64 inside a panel
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;

    extern __shared__ unsigned char smem_raw[];
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int r0 = blk * BT;                               // first key of this CTA
    const int i_begin = p.causal ? r0 / BT : 0;
    const int i_end = (p.Tq + BT - 1) / BT;
    // With tile lists (matrix bias only) the CTA visits the listed query blocks: the count bounds
    // every role's loop, the TMA producer alone reads the list and posts each stage's block index
    // in shared memory (sm.qblk) before the stage's barrier, where the compute threads pick it up.
    int tl_idx = -1;
    if constexpr (LISTS)
        tl_idx = (int)(((p.bias_b0 ? 0 : b) * (p.bias_h0 ? 1 : p.H) + (p.bias_h0 ? 0 : h)) * (int)gridDim.x + blk);
    const int nit = LISTS ? (int)p.tlk_cnt[LISTS ? tl_idx : 0] : max(i_end - i_begin, 0);
    const int nsub = 2 * nit;
    int *status = p.status;

    if (threadIdx.x == 0) {
        mbar_init(&sm.x_full, 1);
        mbar_init(&sm.acc_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.y_full[s], 1);
            mbar_init(&sm.y_empty[s], 1);
            mbar_init(&sm.g1_full[s], 1);
            mbar_init(&sm.g2_full[s], 1);
            mbar_init(&sm.g1_free[s], 1);
            mbar_init(&sm.g2_free[s], 1);
            mbar_init(&sm.p_ready[s], 128);
            mbar_init(&sm.ds_ready[s], 128);
            mbar_init(&sm.bb_full[s], 1);
            mbar_init(&sm.bb_empty[s], 128);
        }
        mbar_init(&sm.dq_full, 1);
        mbar_init(&sm.dq_read, 128);
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

    // Registers move from the helper and read-back warps to the compute warps (the launch gives every
    // thread 65536 / 512 = 128): each role's first instruction resizes its warpgroup.
    if (warp >= 8 && warp < 12) asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    if (warp == 8) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0 && nit > 0) {
            tma_prefetch_desc(&p.mk);
            tma_prefetch_desc(&p.mv);
            tma_prefetch_desc(&p.mq);
            tma_prefetch_desc(&p.mdo);
            if constexpr (BIAS) tma_prefetch_desc(&p.mbias64);
            mbar_expect_tx(&sm.x_full, 2 * TILE_BYTES);
            for (int hh = 0; hh < HALVES; ++hh) {
                tma_load_4d(sm.x1 + hh * PANEL, &p.mk, &sm.x_full, hh * 64, r0, h, b);
                tma_load_4d(sm.x2 + hh * PANEL, &p.mv, &sm.x_full, hh * 64, r0, h, b);
            }
            bool ok = true;
            // the list entry of the next block is fetched while waiting for this block's stage
            const uint16_t *lst = LISTS ? p.tlk_list + (int64_t)tl_idx * p.tl_nqb : nullptr;
            int qb_next = LISTS ? (int)lst[0] : 0;
            for (int it = 0; it < nit; ++it) {
                const int s = it & 1;
                const uint32_t ph = (uint32_t)(it >> 1) & 1u;
                int qb = i_begin + it;
                if constexpr (LISTS) {
                    qb = qb_next;
                    if (it + 1 < nit) qb_next = lst[it + 1];
                }
                ok = mbar_wait(&sm.y_empty[s], ph ^ 1u, status, 71);
                if (!ok) break;
                if constexpr (LISTS) sm.qblk[s] = qb;   // ordered before the arrive below (release), read after the wait on y_full
                mbar_expect_tx(&sm.y_full[s], 2 * TILE_BYTES + (STAGE_STATS ? 2 * BT * 4 : 0));
                const int row = qb * BT;
                if constexpr (STAGE_STATS) {
                    bulk_load_1d(sm.lse_s[s], p.lse2 + (int64_t)bh * p.Tq128 + row, BT * 4, &sm.y_full[s]);
                    bulk_load_1d(sm.dsc_s[s], p.delta_s + (int64_t)bh * p.Tq128 + row, BT * 4, &sm.y_full[s]);
                }
                for (int hh = 0; hh < HALVES; ++hh) {
                    tma_load_4d(sm.y1[s] + hh * PANEL, &p.mq, &sm.y_full[s], hh * 64, row, h, b);
                    tma_load_4d(sm.y2[s] + hh * PANEL, &p.mdo, &sm.y_full[s], hh * 64, row, h, b);
                }
                if constexpr (BIAS) {
                    // sub-tile of sub-block parity sb: queries row + 64 sb .. + 63, keys r0 .. r0 + 127
                    for (int sb = 0; sb < 2 && ok; ++sb) {
                        ok = mbar_wait(&sm.bb_empty[sb], ((uint32_t)it & 1u) ^ 1u, status, 72);
                        if (!ok) break;
                        mbar_expect_tx(&sm.bb_full[sb], BIAS_BYTES);
                        for (int pn = 0; pn < 2; ++pn)
                            tma_load_4d(sm.bias[sb] + pn * (64 * 128), &p.mbias64, &sm.bb_full[sb], r0 + pn * 64,
                                        row + sb * 64, p.bias_h0 ? 0 : h, p.bias_b0 ? 0 : b);
                    }
                    if (!ok) break;
                }
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 9 || warp == 10) {
        // ------------- MMA issuers A1 / A2: the score GEMMs K Q^T and V dO^T -------------
        // One thread can issue an MMA only every ~54 clocks whatever its size, which is as long
        // as these N = 64 MMAs take to run, so each kind of GEMM gets its own issuing thread.
        if (lane == 0 && nit > 0) {
            const bool second = warp == 10;
            constexpr uint32_t idesc_g = make_idesc(BF16, BT, 64, false, false);
            // Descriptors of the operand tiles, encoded once; the loop below only adds offsets.
            const uint64_t dx = make_sdesc(smem_u32(second ? sm.x2 : sm.x1), 16, 1024);
            uint64_t dyk[2];                                 // Q (or dO) per stage, K-major view
#pragma unroll
            for (int s = 0; s < 2; ++s) dyk[s] = make_sdesc(smem_u32(second ? sm.y2[s] : sm.y1[s]), 16, 1024);
            const uint32_t gcol = tbase + (second ? G2_COL : G1_COL);
            uint64_t *full = second ? sm.g2_full : sm.g1_full, *free_ = second ? sm.g2_free : sm.g1_free;
            bool ok = mbar_wait(&sm.x_full, 0, status, 81);
            for (int u = 0; u < nsub && ok; ++u) {
                const int sb = u & 1, it = u >> 1, s = it & 1;
                if (sb == 0) {
                    ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 82);
                    if (!ok) break;
                }
                // the columns are free once the accumulation GEMM of sub-block u - 2 has read them
                if (u >= 2) {
                    ok = mbar_wait(&free_[sb], (uint32_t)(it - 1) & 1u, status, 85);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                // [128 keys] x [64 queries of sub-block u], contraction over channels
                const uint64_t ydu = sdesc_advance(dyk[s], sb * SUB_ROWS);
                const uint32_t dcol = gcol + sb * 64;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * PANEL + (kk % 4) * 32;
                    umma_ss(dcol, sdesc_advance(dx, off), sdesc_advance(ydu, off), idesc_g, kk > 0);
                }
                umma_commit(&full[sb]);
            }
        }
    } else if (warp == 11) {
        // ------------------- MMA issuer B: the accumulation GEMMs -------------------
        // All MMAs that add into dV / dK come from this one thread, in sub-block order, so the
        // order of the floating-point sums is fixed.
        if (lane == 0 && nit > 0) {
            constexpr uint32_t idesc_acc = make_idesc(BF16, BT, D, false, true);
            constexpr uint32_t idesc_dq = make_idesc(BF16, BT, D, true, true);
            const uint64_t ddsm = make_sdesc(smem_u32(sm.dsm), 64 * 128 * 2, 1024);   // two 64-query atoms 16 KB apart
            const uint64_t dkm = make_sdesc(smem_u32(sm.x1), 16, 1024);               // 64 channels: one atom
            uint64_t dy1m[2], dy2m[2];                       // Q / dO per stage, MN-major view
#pragma unroll
            for (int s = 0; s < 2; ++s) {
                dy1m[s] = make_sdesc(smem_u32(sm.y1[s]), PANEL, 1024);
                dy2m[s] = make_sdesc(smem_u32(sm.y2[s]), PANEL, 1024);
            }
            // accumulation GEMM of sub-block u: contraction over its 64 queries (4 steps of 16),
            // packed two per column into the first 32 columns of the sub-block's score columns
            auto issue_acc = [&](int u, uint32_t acc_col, uint32_t a_col, uint64_t yd) {
                const uint64_t ydu = sdesc_advance(yd, (u & 1) * SUB_ROWS);
                const uint32_t acol = tbase + a_col + (u & 1) * 64;
#pragma unroll
                for (int kk = 0; kk < 4; ++kk)
                    umma_ts(tbase + acc_col, acol + kk * 8, sdesc_advance(ydu, kk * 2048), idesc_acc, u > 0 || kk > 0);
            };
            bool ok = true;
            for (int u = 0; u < nsub && ok; ++u) {
                const int sb = u & 1, it = u >> 1, s = it & 1;
                const uint32_t par = (uint32_t)it & 1u;
                if (sb == 0) {
                    ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 87);
                    if (!ok) break;
                }
                ok = mbar_wait(&sm.p_ready[sb], par, status, 83);
                if (!ok) break;
                tc_fence_after_sync();
                issue_acc(u, ACC1_COL, G1_COL, dy2m[s]);            // dV += P^T dO
                tc_fence_before_sync();
                mbar_arrive(&sm.g1_free[sb]);   // issued, not finished: the tensor pipe runs MMAs in issue order
                ok = mbar_wait(&sm.ds_ready[sb], par, status, 84);
                if (!ok) break;
                tc_fence_after_sync();
                issue_acc(u, ACC2_COL, G2_COL, dy1m[s]);            // dK += dS^T Q
                tc_fence_before_sync();
                mbar_arrive(&sm.g2_free[sb]);
                if (sb == 1) {
                    umma_commit(&sm.y_empty[s]);                     // both sub-blocks of this block consumed
                    // dQ partial tile of this block: [128 queries x 64 channels] = dS [queries x keys] K, with
                    // A = dS^T as the compute threads left it in shared memory ([key][query], MN-major, one
                    // 64-query atom per sub-block) and B = the resident K tile ([key][channel], MN-major).
                    // Its columns are free once the read-back warps hold the previous block's tile.
                    if (it >= 1) {
                        ok = mbar_wait(&sm.dq_read, (uint32_t)(it - 1) & 1u, status, 121);
                        if (!ok) break;
                        tc_fence_after_sync();
                    }
#pragma unroll
                    for (int kk = 0; kk < BT / 16; ++kk)
                        umma_ss(tbase + DQ_COL, sdesc_advance(ddsm, kk * 2048), sdesc_advance(dkm, kk * 2048), idesc_dq, kk > 0);
                    umma_commit(&sm.dq_full);
                }
            }
            umma_commit(&sm.acc_full);
        }
    } else if (warp >= 12) {
        // ------------- read-back warps: dQ partial tiles -> fp32 accumulator in global memory -------------
        // Thread = query row of the block.  The accumulator of a (batch, head) is laid out
        // [channel / 4][query][channel % 4], so a warp's 16-byte vector reduction covers 512
        // contiguous bytes.  These warps take the stalls of the reduction traffic.
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        const int row_l = (warp & 3) * 32 + lane;
        const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        float *acc_bh = p.dq_acc + (int64_t)bh * (D / 4) * p.Tq128 * 4;
        bool ok = true;
        for (int it = 0; it < nit && ok; ++it) {
            ok = mbar_wait(&sm.dq_full, (uint32_t)it & 1u, status, 122);
            if (!ok) break;
            tc_fence_after_sync();
            float *dst = acc_bh + ((int64_t)(i_begin + it) * BT + row_l) * 4;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                tmem_ld32(lane_base + DQ_COL + c * 32, r);
                tmem_wait_ld();
                if (c == 1) {
                    tc_fence_before_sync();
                    mbar_arrive(&sm.dq_read);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + (int64_t)(c * 8 + i) * p.Tq128 * 4),
                                 "f"(__uint_as_float(r[4 * i])), "f"(__uint_as_float(r[4 * i + 1])),
                                 "f"(__uint_as_float(r[4 * i + 2])), "f"(__uint_as_float(r[4 * i + 3]))
                                 : "memory");
            }
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        asm volatile("setmaxnreg.inc.sync.aligned.u32 184;");
        // Warps 0-3 own the even sub-blocks, warps 4-7 the odd ones: each thread handles one
        // key row and all 64 queries of its sub-block, and the two groups run half a period
        // apart, so one group's exponentials overlap the other's tensor-memory round trips.
        const int row_l = (warp & 3) * 32 + lane;          // key row of the tile == TMEM lane
        const int sb = warp >> 2;                          // sub-block parity this warp group owns
        const int half = sb;                               // epilogue: which half of the channels
        const int row = r0 + row_l;
        const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        const bool cta_key_tail = r0 + BT > p.Tk;
        const uint32_t col = sb * 64;                      // this group's columns inside G1 / G2
        // vector bias: this thread's key has one value for every query, times log2(e)
        float bk2 = 0.f;
        if constexpr (BIASM == 2) {
            if (row < p.Tk) {
                const char *bias_bh = reinterpret_cast<const char *>(p.bias) +
                                      ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : 2);
                bk2 = (p.bias_f32 ? reinterpret_cast<const float *>(bias_bh)[row]
                                  : to_f32<T>(reinterpret_cast<const T *>(bias_bh)[row])) * LOG2E;
            }
        }

        bool ok = true;
        for (int it = 0; it < nit; ++it) {
            const uint32_t par = (uint32_t)it & 1u;
            const int s = it & 1;
            int blk0 = (i_begin + it) * BT;
            if constexpr (LISTS) {
                // the block's index is posted with its tiles
                ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 90);
                if (!ok) break;
                blk0 = sm.qblk[s] * BT;
            }
            const int c0 = blk0 + sb * 64;                 // first query of the sub-block
            const bool slow = cta_key_tail || (p.causal && blk0 == r0);
            // row statistics of this sub-block's 64 queries: staged in shared memory, else from global
            const float *lse_f = STAGE_STATS ? &sm.lse_s[s][sb * 64] : p.lse2 + (int64_t)bh * p.Tq128 + c0;
            const float *dsc_f = STAGE_STATS ? &sm.dsc_s[s][sb * 64] : p.delta_s + (int64_t)bh * p.Tq128 + c0;
            const float4 *lse4 = reinterpret_cast<const float4 *>(lse_f);
            const float4 *dsc4 = reinterpret_cast<const float4 *>(dsc_f);
            float pv[64];

            if constexpr (!LISTS) {
                // row statistics of this block have landed
                ok = mbar_wait(&sm.y_full[s], (uint32_t)(it >> 1) & 1u, status, 90);
                if (!ok) break;
            }

            // x0[i] = bias * log2(e) - lse * log2(e) of query i (only -lse without a bias), formed
            // before the scores are waited for
            float x0[BIAS ? 64 : 1];
            if constexpr (BIAS) {
                ok = mbar_wait(&sm.bb_full[sb], (uint32_t)it & 1u, status, 94);
                if (!ok) break;
                // this thread's key column of the sub-tile: panel = key / 64, 16-byte chunk index
                // XOR (query mod 8) inside the 128-byte row of query i
                const unsigned char *colp = sm.bias[sb] + (row_l >> 6) * (64 * 128) + (row_l & 7) * 2;
                const int kc = (row_l & 63) >> 3;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 l = lse4[i];
                    const float lv[4] = {l.x, l.y, l.z, l.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int qi = 4 * i + e;
                        const float bvl = to_f32<T>(*reinterpret_cast<const T *>(colp + qi * 128 + ((kc ^ (qi & 7)) << 4)));
                        x0[qi] = fmaf(bvl, LOG2E, -lv[e]);
                    }
                }
            }
            ok = mbar_wait(&sm.g1_full[sb], par, status, 91);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t ra[32], rb[32];
                tmem_ld32(lane_base + G1_COL + col, ra);
                tmem_ld32(lane_base + G1_COL + col + 32, rb);
                tmem_wait_ld();
                if (!slow) {
                    if constexpr (BIAS) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            pv[i] = ex2b(fmaf(__uint_as_float(ra[i]), p.scale_log2, x0[i]));
                            pv[32 + i] = ex2b(fmaf(__uint_as_float(rb[i]), p.scale_log2, x0[32 + i]));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 l = lse4[i];
                            pv[4 * i + 0] = ex2b(fmaf(__uint_as_float(ra[4 * i + 0]), p.scale_log2, bk2 - l.x));
                            pv[4 * i + 1] = ex2b(fmaf(__uint_as_float(ra[4 * i + 1]), p.scale_log2, bk2 - l.y));
                            pv[4 * i + 2] = ex2b(fmaf(__uint_as_float(ra[4 * i + 2]), p.scale_log2, bk2 - l.z));
                            pv[4 * i + 3] = ex2b(fmaf(__uint_as_float(ra[4 * i + 3]), p.scale_log2, bk2 - l.w));
                        }
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            const float4 l = lse4[8 + i];
                            pv[32 + 4 * i + 0] = ex2b(fmaf(__uint_as_float(rb[4 * i + 0]), p.scale_log2, bk2 - l.x));
                            pv[32 + 4 * i + 1] = ex2b(fmaf(__uint_as_float(rb[4 * i + 1]), p.scale_log2, bk2 - l.y));
                            pv[32 + 4 * i + 2] = ex2b(fmaf(__uint_as_float(rb[4 * i + 2]), p.scale_log2, bk2 - l.z));
                            pv[32 + 4 * i + 3] = ex2b(fmaf(__uint_as_float(rb[4 * i + 3]), p.scale_log2, bk2 - l.w));
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 64; ++i) {
                        const int qi = c0 + i;
                        const bool masked = row >= p.Tk || qi >= p.Tq || (p.causal && row > qi);
                        const float sv = __uint_as_float(i < 32 ? ra[i & 31] : rb[i & 31]);
                        const float off = BIAS ? x0[BIAS ? i : 0] : bk2 - lse_f[i];
                        pv[i] = masked ? 0.f : ex2b(fmaf(sv, p.scale_log2, off));
                    }
                }
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) pk[i] = pack16b<BF16>(pv[2 * i], pv[2 * i + 1]);
                tmem_st32(lane_base + G1_COL + col, pk);
                tmem_wait_st();
            }
            // P, which depends on every bias value read above, is stored: the bias stage is free
            if constexpr (BIAS) mbar_arrive(&sm.bb_empty[sb]);
            tc_fence_before_sync();
            mbar_arrive(&sm.p_ready[sb]);

            ok = mbar_wait(&sm.g2_full[sb], par, status, 92);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t ga[32], gb[32];
                tmem_ld32(lane_base + G2_COL + col, ga);
                tmem_ld32(lane_base + G2_COL + col + 32, gb);
                tmem_wait_ld();
                uint32_t pk[32];
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float4 dd = dsc4[i];
                    const uint32_t *g = i < 8 ? ga : gb;
                    const int j = (i & 7) * 4;
                    const float a0 = pv[4 * i + 0] * fmaf(__uint_as_float(g[j + 0]), p.scale, -dd.x);
                    const float a1 = pv[4 * i + 1] * fmaf(__uint_as_float(g[j + 1]), p.scale, -dd.y);
                    const float a2 = pv[4 * i + 2] * fmaf(__uint_as_float(g[j + 2]), p.scale, -dd.z);
                    const float a3 = pv[4 * i + 3] * fmaf(__uint_as_float(g[j + 3]), p.scale, -dd.w);
                    pk[2 * i] = pack16b<BF16>(a0, a1);
                    pk[2 * i + 1] = pack16b<BF16>(a2, a3);
                }
                tmem_st32(lane_base + G2_COL + col, pk);
                // dS^T also goes to shared memory for the dQ partial GEMM, once the GEMM of the previous
                // block has read it: this key's 64 queries are one 128-byte row, 16-byte chunk c = queries
                // 8c .. 8c + 7, 128-byte swizzle
                if (it >= 1) {
                    ok = mbar_wait(&sm.dq_full, (uint32_t)(it - 1) & 1u, status, 123);
                    if (!ok) break;
                }
                unsigned char *ds_row = sm.dsm + sb * (64 * 128 * 2) + row_l * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4 *>(ds_row + ((c ^ (row_l & 7)) << 4)) =
                        make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
                fence_proxy_async_smem();
                tmem_wait_st();
            }
            tc_fence_before_sync();
            mbar_arrive(&sm.ds_ready[sb]);
        }

        // epilogue: dV, dK -> global
        if (ok && nit > 0) ok = mbar_wait(&sm.acc_full, 0, status, 93);
        tc_fence_after_sync();
        if (ok) {
#pragma unroll
            for (int o = 0; o < 2; ++o) {
                T *base = reinterpret_cast<T *>(o == 0 ? p.out1 : p.out2);
                const int64_t sb_ = o == 0 ? p.o1_sb : p.o2_sb, sh = o == 0 ? p.o1_sh : p.o2_sh,
                              sn = o == 0 ? p.o1_sn : p.o2_sn;
                T *orow = base + (int64_t)b * sb_ + (int64_t)h * sh + (int64_t)row * sn;
                const uint32_t acc_col = o == 0 ? ACC1_COL : ACC2_COL;
#pragma unroll 1
                for (int c = 0; c < D / 64; ++c) {
                    const int cc = half * (D / 2) + c * 32;
                    uint32_t r[32];
                    if (nit > 0) {
                        tmem_ld32(lane_base + acc_col + cc, r);
                        tmem_wait_ld();
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = 0u;
                    }
                    if (row < p.Tk) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 v;
                            v.x = pack16b<BF16>(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
                            v.y = pack16b<BF16>(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
                            v.z = pack16b<BF16>(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
                            v.w = pack16b<BF16>(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
                            *reinterpret_cast<uint4 *>(orow + cc + i) = v;
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
// dQ without bias, pipelined.  One CTA per 128-query tile, looping over key blocks:
//   S = Q K^T, dP = dO V^T (SS MMAs), P = exp2(S * scale * log2e - lse2) in registers,
//   dS = P * (dP * scale - delta_s) packed into the dP columns, dQ += dS K (TS MMA).
// What bounds the loop is latency, not arithmetic, so every hand-off gets slack:
//  * K tiles sit in a ring of three (a tile is needed from its score GEMM until its dQ GEMM,
//    one whole block later, so with two the next load would start only when it is already
//    needed); V tiles, used by one GEMM only, in a ring of two.
//  * The compute warps form dS of block i and, in the same pass, P of block i + 1 (which stays
//    in registers), so the exponentials overlap the dS arithmetic.  The dP / dS columns are
//    double-buffered (tensor-memory columns 128 and 384): dP of the next block is ready
//    while the dQ GEMM still reads dS of this one; S runs two blocks ahead of dS.
//  * Two MMA-issuing threads (score GEMMs / dQ GEMMs): one thread can issue an MMA only
//    every ~54 clocks whatever its size.  All dQ MMAs come from one thread, in block order,
//    so the order of the floating-point sums is fixed.
// ---------------------------------------------------------------------------
template <int D>
struct alignas(1024) DqPipeSmem {
    unsigned char xq[BT * D * 2], xdo[BT * D * 2];           // Q, dO of this CTA's query tile
    unsigned char k[3][BT * D * 2], v[2][BT * D * 2];
    uint64_t x_full, g1_full, s_read, ds_ready, acc_full;
    uint64_t k_full[3], k_empty[3], v_full[2], v_empty[2];
    uint64_t g2_full[2], g2_free[2];                         // per dP / dS column buffer
    uint32_t tmem_base;
};
constexpr int DQ_PIPE_THREADS = 352;   // 8 compute warps, TMA producer, two MMA issuers

// VEC: a vector bias (one value per key) is added to the scores; each compute thread fetches the
// values of its 64 keys per block (the same for every query row, so they come from L1).
template <int D, bool BF16, bool VEC>
__global__ void __launch_bounds__(DQ_PIPE_THREADS, 1) attn_bwd_dq_pipe(const __grid_constant__ BwdTmaParams p) {
    constexpr int HALVES = D / 64;
    constexpr uint32_t PANEL = 128 * 64 * 2;
    constexpr uint32_t TILE_BYTES = BT * D * 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t G1_COL = 0, G2A_COL = 128, ACC_COL = 256, G2B_COL = 384;
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;

    extern __shared__ unsigned char smem_raw[];
    DqPipeSmem<D> &sm = *reinterpret_cast<DqPipeSmem<D> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int r0 = blk * BT;                               // first query of this CTA
    const int i_end = ((p.causal ? min(p.Tk, r0 + BT) : p.Tk) + BT - 1) / BT;
    const int nit = max(i_end, 0);
    int *status = p.status;

    if (threadIdx.x == 0) {
        mbar_init(&sm.x_full, 1);
        mbar_init(&sm.g1_full, 1);
        mbar_init(&sm.s_read, 256);
        mbar_init(&sm.ds_ready, 256);
        mbar_init(&sm.acc_full, 1);
        for (int s = 0; s < 3; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
            mbar_init(&sm.g2_full[s], 1);
            mbar_init(&sm.g2_free[s], 1);
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
            tma_prefetch_desc(&p.mq);
            tma_prefetch_desc(&p.mdo);
            tma_prefetch_desc(&p.mk);
            tma_prefetch_desc(&p.mv);
            mbar_expect_tx(&sm.x_full, 2 * TILE_BYTES);
            for (int hh = 0; hh < HALVES; ++hh) {
                tma_load_4d(sm.xq + hh * PANEL, &p.mq, &sm.x_full, hh * 64, r0, h, b);
                tma_load_4d(sm.xdo + hh * PANEL, &p.mdo, &sm.x_full, hh * 64, r0, h, b);
            }
            bool ok = true;
            int ks = 0;
            uint32_t kph = 0;                              // phase of the K ring slot's previous use
            for (int it = 0; it < nit; ++it) {
                const int row = it * BT;
                ok = mbar_wait(&sm.k_empty[ks], kph ^ 1u, status, 41);
                if (!ok) break;
                mbar_expect_tx(&sm.k_full[ks], TILE_BYTES);
                for (int hh = 0; hh < HALVES; ++hh)
                    tma_load_4d(sm.k[ks] + hh * PANEL, &p.mk, &sm.k_full[ks], hh * 64, row, h, b);
                if (++ks == 3) { ks = 0; kph ^= 1u; }
                const int vs = it & 1;
                ok = mbar_wait(&sm.v_empty[vs], ((uint32_t)(it >> 1) & 1u) ^ 1u, status, 42);
                if (!ok) break;
                mbar_expect_tx(&sm.v_full[vs], TILE_BYTES);
                for (int hh = 0; hh < HALVES; ++hh)
                    tma_load_4d(sm.v[vs] + hh * PANEL, &p.mv, &sm.v_full[vs], hh * 64, row, h, b);
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 9) {
        // ---------------------- MMA issuer A: the score GEMMs ----------------------
        if (lane == 0 && nit > 0) {
            constexpr uint32_t idesc_g = make_idesc(BF16, BT, BT, false, false);
            const uint64_t dxq = make_sdesc(smem_u32(sm.xq), 16, 1024), dxdo = make_sdesc(smem_u32(sm.xdo), 16, 1024);
            auto issue_g = [&](uint32_t col, uint64_t xd, uint64_t yd) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * PANEL + (kk % 4) * 32;
                    umma_ss(tbase + col, sdesc_advance(xd, off), sdesc_advance(yd, off), idesc_g, kk > 0);
                }
            };
            // S of block j (K ring slot and phase advance with j)
            int ks = 0;
            uint32_t kph = 0;
            auto issue_g1 = [&](int j) -> bool {
                if (!mbar_wait(&sm.k_full[ks], kph, status, 52)) return false;
                // the score columns are free once the compute warps have read S of block j - 1
                if (j >= 1 && !mbar_wait(&sm.s_read, (uint32_t)(j - 1) & 1u, status, 53)) return false;
                tc_fence_after_sync();
                issue_g(G1_COL, dxq, make_sdesc(smem_u32(sm.k[ks]), 16, 1024));
                umma_commit(&sm.g1_full);
                if (++ks == 3) { ks = 0; kph ^= 1u; }
                return true;
            };
            // dP of block j into dP buffer j & 1
            auto issue_g2 = [&](int j) -> bool {
                const int vs = j & 1;
                if (!mbar_wait(&sm.v_full[vs], (uint32_t)(j >> 1) & 1u, status, 54)) return false;
                // the buffer is free once the dQ GEMM of block j - 2 has read dS from it
                if (j >= 2 && !mbar_wait(&sm.g2_free[vs], (uint32_t)((j >> 1) - 1) & 1u, status, 55)) return false;
                tc_fence_after_sync();
                issue_g(vs ? G2B_COL : G2A_COL, dxdo, make_sdesc(smem_u32(sm.v[vs]), 16, 1024));
                umma_commit(&sm.g2_full[vs]);
                umma_commit(&sm.v_empty[vs]);
                return true;
            };
            // Both kinds of GEMM run ahead of the compute warps, which in iteration `it` form dS
            // of block it and P of block it + 1: dP one block ahead, S two blocks ahead.
            bool ok = mbar_wait(&sm.x_full, 0, status, 51);
            if (ok) ok = issue_g1(0);
            if (ok) ok = issue_g2(0);
            if (ok && nit > 1) ok = issue_g1(1);
            for (int it = 0; it < nit && ok; ++it) {
                if (it + 1 < nit) ok = issue_g2(it + 1);
                if (ok && it + 2 < nit) ok = issue_g1(it + 2);
            }
        }
    } else if (warp == 10) {
        // ---------------------- MMA issuer B: the dQ GEMMs ----------------------
        if (lane == 0 && nit > 0) {
            constexpr uint32_t idesc_acc = make_idesc(BF16, BT, D, false, true);
            bool ok = true;
            int ks = 0;
            uint32_t kph = 0;
            for (int it = 0; it < nit && ok; ++it) {
                ok = mbar_wait(&sm.k_full[ks], kph, status, 56);
                if (!ok) break;
                ok = mbar_wait(&sm.ds_ready, (uint32_t)it & 1u, status, 57);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t dkm = make_sdesc(smem_u32(sm.k[ks]), PANEL, 1024);   // K as [key][channel], MN-major
                // each half of the compute threads packed its 64 keys into the first 32 of its own 64 columns
#pragma unroll
                for (int kk = 0; kk < BT / 16; ++kk)
                    umma_ts(tbase + ACC_COL, tbase + ((it & 1) ? G2B_COL : G2A_COL) + (kk >> 2) * 64 + (kk & 3) * 8,
                            sdesc_advance(dkm, kk * 2048), idesc_acc, it > 0 || kk > 0);
                tc_fence_before_sync();
                mbar_arrive(&sm.g2_free[it & 1]);   // issued, not finished: the tensor pipe runs MMAs in issue order
                umma_commit(&sm.k_empty[ks]);
                if (++ks == 3) { ks = 0; kph ^= 1u; }
            }
            umma_commit(&sm.acc_full);
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        const int row_l = (warp & 3) * 32 + lane;          // query row of the tile == TMEM lane
        const int half = warp >> 2;                        // which 64 of the block's 128 keys
        const int row = r0 + row_l;
        const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        // rows past Tq hold +inf / 0, so they yield P = 0
        const float lse_row = p.lse2[(int64_t)bh * p.Tq128 + row];
        const float dsc_row = p.delta_s[(int64_t)bh * p.Tq128 + row];

        const char *bias_bh = nullptr;
        if constexpr (VEC)
            bias_bh = reinterpret_cast<const char *>(p.bias) +
                      ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : 2);
        // off[i] = bias * log2(e) - lse * log2(e) for the 32 keys starting at column c of this
        // thread's 64 in block j (just -lse without a bias); keys past the end read as bias 0
        auto offsets = [&](int j, int c, float *off) {
            if constexpr (VEC) {
                const int k0 = j * BT + half * 64 + c;
                if (!p.bias_f32 && p.bias_vec && k0 + 32 <= p.Tk) {
                    const T *src = reinterpret_cast<const T *>(bias_bh) + k0;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        const Vec<T, 8> v8 = load_vec<T, 8>(src + 8 * q4);
#pragma unroll
                        for (int e = 0; e < 8; ++e) off[8 * q4 + e] = fmaf(to_f32<T>(v8.v[e]), LOG2E, -lse_row);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float bvl = 0.f;
                        if (k0 + i < p.Tk)
                            bvl = p.bias_f32 ? reinterpret_cast<const float *>(bias_bh)[k0 + i]
                                             : to_f32<T>(reinterpret_cast<const T *>(bias_bh)[k0 + i]);
                        off[i] = fmaf(bvl, LOG2E, -lse_row);
                    }
                }
            }
        };
        // P of block j from its scores (32 columns starting at column c of this thread's 64)
        auto p_from_s = [&](const uint32_t (&r)[32], float *pv, int j, int c) {
            const int blk0 = j * BT;
            float off[VEC ? 32 : 1];
            offsets(j, c, off);
            // blocks that need per-element masking: the diagonal blocks under the causal mask
            // and the block touching the end of the keys
            const bool slow = (p.causal && blk0 + BT > r0) || blk0 + BT > p.Tk;
            if (!slow) {
#pragma unroll
                for (int i = 0; i < 32; ++i)
                    pv[i] = ex2b(fmaf(__uint_as_float(r[i]), p.scale_log2, VEC ? off[VEC ? i : 0] : -lse_row));
            } else {
                const int c0 = blk0 + half * 64 + c;
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int kj = c0 + i;
                    const bool masked = kj >= p.Tk || row >= p.Tq || (p.causal && kj > row);
                    pv[i] = masked ? 0.f : ex2b(fmaf(__uint_as_float(r[i]), p.scale_log2, VEC ? off[VEC ? i : 0] : -lse_row));
                }
            }
        };

        bool ok = true;
        float pv[64];
        // prologue: P of block 0
        if (nit > 0) {
            ok = mbar_wait(&sm.g1_full, 0, status, 60);
            if (ok) {
                tc_fence_after_sync();
                uint32_t ra[32], rb[32];
                tmem_ld32(lane_base + G1_COL + half * 64, ra);
                tmem_ld32(lane_base + G1_COL + half * 64 + 32, rb);
                tmem_wait_ld();
                tc_fence_before_sync();
                mbar_arrive(&sm.s_read);                   // P stays in registers: the columns are free
                p_from_s(ra, pv, 0, 0);
                p_from_s(rb, pv + 32, 0, 32);
            }
        }
        // Block it: dS from P (registers) and dP; in the same pass, P of block it + 1 from its
        // scores, so the exponentials (MUFU) overlap the dS arithmetic (FMA pipe) and the waits.
        for (int it = 0; it < nit && ok; ++it) {
            const bool next = it + 1 < nit;
            const uint32_t dcol = ((it & 1) ? G2B_COL : G2A_COL) + half * 64;
            const bool slow_next = (p.causal && (it + 1) * BT + BT > r0) || (it + 1) * BT + BT > p.Tk;
            ok = mbar_wait(&sm.g2_full[it & 1], (uint32_t)(it >> 1) & 1u, status, 62);
            if (!ok) break;
            if (next) {
                ok = mbar_wait(&sm.g1_full, (uint32_t)(it + 1) & 1u, status, 61);
                if (!ok) break;
            }
            tc_fence_after_sync();
            const uint32_t scol = G1_COL + half * 64;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t ga[32], ra[32];
                tmem_ld32(lane_base + dcol + c * 32, ga);
                if (next) tmem_ld32(lane_base + scol + c * 32, ra);
                tmem_wait_ld();
                if (c == 1 && next) {                      // all of S read: the next score GEMM may start
                    tc_fence_before_sync();
                    mbar_arrive(&sm.s_read);
                }
                uint32_t pk[16];
                if (next && !slow_next) {
                    float off[VEC ? 32 : 1];
                    offsets(it + 1, 32 * c, off);
                    // element by element, so that the exponentials of the next block (MUFU) and
                    // the dS arithmetic of this one (FMA pipe) issue side by side
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float a0 = pv[32 * c + 2 * i] * fmaf(__uint_as_float(ga[2 * i]), p.scale, -dsc_row);
                        const float a1 = pv[32 * c + 2 * i + 1] * fmaf(__uint_as_float(ga[2 * i + 1]), p.scale, -dsc_row);
                        pv[32 * c + 2 * i] = ex2b(fmaf(__uint_as_float(ra[2 * i]), p.scale_log2,
                                                       VEC ? off[VEC ? 2 * i : 0] : -lse_row));
                        pv[32 * c + 2 * i + 1] = ex2b(fmaf(__uint_as_float(ra[2 * i + 1]), p.scale_log2,
                                                           VEC ? off[VEC ? 2 * i + 1 : 0] : -lse_row));
                        pk[i] = pack16b<BF16>(a0, a1);
                    }
                    // packed dS of chunk c goes to columns [c*16, c*16+16) of this thread's 64, all read already
                    tmem_st16(lane_base + dcol + c * 16, pk);
                } else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float a0 = pv[32 * c + 2 * i] * fmaf(__uint_as_float(ga[2 * i]), p.scale, -dsc_row);
                        const float a1 = pv[32 * c + 2 * i + 1] * fmaf(__uint_as_float(ga[2 * i + 1]), p.scale, -dsc_row);
                        pk[i] = pack16b<BF16>(a0, a1);
                    }
                    tmem_st16(lane_base + dcol + c * 16, pk);
                    if (next) p_from_s(ra, pv + 32 * c, it + 1, 32 * c);
                }
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.ds_ready);
        }

        // epilogue: dQ -> global
        if (ok && nit > 0) ok = mbar_wait(&sm.acc_full, 0, status, 63);
        tc_fence_after_sync();
        if (ok) {
            T *orow = reinterpret_cast<T *>(p.out1) + (int64_t)b * p.o1_sb + (int64_t)h * p.o1_sh + (int64_t)row * p.o1_sn;
#pragma unroll 1
            for (int c = 0; c < D / 64; ++c) {
                const int col = half * (D / 2) + c * 32;
                uint32_t r[32];
                if (nit > 0) {
                    tmem_ld32(lane_base + ACC_COL + col, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                }
                if (row < p.Tq) {
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

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// dQ with a matrix bias staged by TMA.  One CTA per 128-query tile, looping over key blocks:
//   S = Q K^T, dP = dO V^T, P = exp2(S * scale * log2e + bias * log2e - lse2) in registers,
//   dS = P * (dP * scale - delta_s) packed into the dP columns, dQ += dS K.
// All three GEMMs take their A operand from TENSOR MEMORY: Q and dO, which are the same for
// every key block, are written there once (packed 16-bit pairs) by the compute threads, straight
// from global memory, so the Q / dO tiles need no shared memory and two 128 x 128 bias tiles
// fit beside the K and V rings.
// Tensor memory (512 columns): S at 0, dP / dS at 128, dQ accumulator at 256, Q at 384, dO at 448.
// S and dP are single-buffered; the loop keeps the tensor pipe fed like this:
//   compute, block it:  dS(it) from P(it) (registers) and dP(it)            -> ds_ready
//                       P(it+1) from S(it+1) and bias tile it+1, registers  -> s_read   (while the
//                       pipe runs dQ(it), dP(it+1) and S(it+2))
//   issuer A:           dP(j) once dQ(j-1) has been issued (MMAs run in issue order, so it reads
//                       dS before dP(j) overwrites it); S(j) once S(j-1) has been read
//   issuer B:           dQ(j) once dS(j) is in place; all dQ MMAs come from this one thread, in
//                       block order, so the order of the floating-point sums is fixed.
// A bias stage is handed back when dS of its block has been stored (every value read from the
// stage has been consumed by then).
// ---------------------------------------------------------------------------
template <int D>
struct alignas(1024) DqBiasSmem {
    unsigned char k[3][BT * D * 2], v[2][BT * D * 2];
    unsigned char bias[2][BT * BT * 2];
    uint64_t a_ready, g1_full, g2_full, s_read, ds_ready, g2_free, acc_full;
    uint64_t k_full[3], k_empty[3], v_full[2], v_empty[2], bb_full[2], bb_empty[2];
    uint32_t tmem_base;
};

// VEC: the bias is a vector (one value per key, 16-bit, 16-byte addressable, key count a multiple of 8):
// the producer stages the block's 128 values (256 bytes) with one bulk copy instead of a 32 KB tile, and
// every compute thread reads its 64 from shared memory (the same addresses in all threads: broadcasts).
template <int D, bool BF16, bool DBIAS, bool LISTS, bool VEC>
__global__ void __launch_bounds__(DQ_PIPE_THREADS, 1) attn_bwd_dq_bias(const __grid_constant__ BwdTmaParams p,
                                                                       const void *q_base, const void *do_base,
                                                                       int64_t q_sb, int64_t q_sh, int64_t q_sn,
                                                                       int64_t do_sb, int64_t do_sh, int64_t do_sn) {
    constexpr int HALVES = D / 64;
    constexpr uint32_t PANEL = 128 * 64 * 2;
    constexpr uint32_t TILE_BYTES = BT * D * 2;
    constexpr uint32_t BIAS_BYTES = BT * BT * 2;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t G1_COL = 0, G2_COL = 128, ACC_COL = 256, QA_COL = 384, DOA_COL = 448;
    constexpr int ACOLS = D / 4;                           // packed columns each compute thread fills per operand
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;

    extern __shared__ unsigned char smem_raw[];
    DqBiasSmem<D> &sm = *reinterpret_cast<DqBiasSmem<D> *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.x, bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int r0 = blk * BT;                               // first query of this CTA
    const int i_end = ((p.causal ? min(p.Tk, r0 + BT) : p.Tk) + BT - 1) / BT;
    int nit = max(i_end, 0);
    // key blocks to visit when the bias came with tile lists (an instantiation of its own): the
    // others hold only masked values
    const uint16_t *tl = nullptr;
    if constexpr (LISTS) {
        const int64_t slice = (int64_t)(p.bias_b0 ? 0 : b) * (p.bias_h0 ? 1 : p.H) + (p.bias_h0 ? 0 : h);
        const int64_t idx = slice * gridDim.x + blk;
        tl = p.tlq_list + idx * p.tl_nkb;
        nit = p.tlq_cnt[idx];
    }
    int *status = p.status;

    if (threadIdx.x == 0) {
        mbar_init(&sm.a_ready, 256);
        mbar_init(&sm.g1_full, 1);
        mbar_init(&sm.g2_full, 1);
        mbar_init(&sm.s_read, 256);
        mbar_init(&sm.ds_ready, 256);
        mbar_init(&sm.g2_free, 1);
        mbar_init(&sm.acc_full, 1);
        for (int s = 0; s < 3; ++s) {
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
            mbar_init(&sm.bb_full[s], 1);
            mbar_init(&sm.bb_empty[s], 256);
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
            tma_prefetch_desc(&p.mk);
            tma_prefetch_desc(&p.mv);
            if constexpr (!VEC) tma_prefetch_desc(&p.mbias);
            bool ok = true;
            int ks = 0;
            uint32_t kph = 0;                              // phase of the K ring slot's previous use
            for (int it = 0; it < nit; ++it) {
                const int row = (LISTS ? (int)tl[it] : it) * BT;
                ok = mbar_wait(&sm.k_empty[ks], kph ^ 1u, status, 41);
                if (!ok) break;
                mbar_expect_tx(&sm.k_full[ks], TILE_BYTES);
                for (int hh = 0; hh < HALVES; ++hh)
                    tma_load_4d(sm.k[ks] + hh * PANEL, &p.mk, &sm.k_full[ks], hh * 64, row, h, b);
                if (++ks == 3) { ks = 0; kph ^= 1u; }
                const int vs = it & 1;
                // bias tile of block it: rows = this CTA's queries, columns = the block's keys
                ok = mbar_wait(&sm.bb_empty[vs], ((uint32_t)(it >> 1) & 1u) ^ 1u, status, 43);
                if (!ok) break;
                if constexpr (VEC) {
                    const uint32_t nbytes = (uint32_t)min(BT, p.Tk - row) * 2u;       // a multiple of 16
                    mbar_expect_tx(&sm.bb_full[vs], nbytes);
                    bulk_load_1d(sm.bias[vs], reinterpret_cast<const char *>(p.bias) +
                                                  ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh + row) * 2, nbytes, &sm.bb_full[vs]);
                } else {
                    mbar_expect_tx(&sm.bb_full[vs], BIAS_BYTES);
                    for (int pn = 0; pn < 2; ++pn)
                        tma_load_4d(sm.bias[vs] + pn * (BT * 128), &p.mbias, &sm.bb_full[vs], row + pn * 64, r0,
                                    p.bias_h0 ? 0 : h, p.bias_b0 ? 0 : b);
                }
                ok = mbar_wait(&sm.v_empty[vs], ((uint32_t)(it >> 1) & 1u) ^ 1u, status, 42);
                if (!ok) break;
                mbar_expect_tx(&sm.v_full[vs], TILE_BYTES);
                for (int hh = 0; hh < HALVES; ++hh)
                    tma_load_4d(sm.v[vs] + hh * PANEL, &p.mv, &sm.v_full[vs], hh * 64, row, h, b);
            }
            if (!ok)
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
        }
    } else if (warp == 9) {
        // ---------------------- MMA issuer A: the score GEMMs ----------------------
        if (lane == 0 && nit > 0) {
            constexpr uint32_t idesc_g = make_idesc(BF16, BT, BT, false, false);
            // [128 queries, A in tensor memory] x [128 keys of the tile at `yd`], contraction over channels
            auto issue_g = [&](uint32_t col, uint32_t a_col, uint64_t yd) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * PANEL + (kk % 4) * 32;
                    umma_ts(tbase + col, tbase + a_col + kk * 8, sdesc_advance(yd, off), idesc_g, kk > 0);
                }
            };
            int ks = 0;
            uint32_t kph = 0;
            // S of block j (K ring slot and phase advance with j)
            auto issue_g1 = [&](int j) -> bool {
                if (!mbar_wait(&sm.k_full[ks], kph, status, 52)) return false;
                // the score columns are free once the compute warps have read S of block j - 1
                if (j >= 1 && !mbar_wait(&sm.s_read, (uint32_t)(j - 1) & 1u, status, 53)) return false;
                tc_fence_after_sync();
                issue_g(G1_COL, QA_COL, make_sdesc(smem_u32(sm.k[ks]), 16, 1024));
                umma_commit(&sm.g1_full);
                if (++ks == 3) { ks = 0; kph ^= 1u; }
                return true;
            };
            // dP of block j
            auto issue_g2 = [&](int j) -> bool {
                const int vs = j & 1;
                if (!mbar_wait(&sm.v_full[vs], (uint32_t)(j >> 1) & 1u, status, 54)) return false;
                // the columns are free once the dQ GEMM of block j - 1 (which reads dS from them) is issued
                if (j >= 1 && !mbar_wait(&sm.g2_free, (uint32_t)(j - 1) & 1u, status, 55)) return false;
                tc_fence_after_sync();
                issue_g(G2_COL, DOA_COL, make_sdesc(smem_u32(sm.v[vs]), 16, 1024));
                umma_commit(&sm.g2_full);
                umma_commit(&sm.v_empty[vs]);
                return true;
            };
            bool ok = mbar_wait(&sm.a_ready, 0, status, 51);       // Q and dO are in tensor memory
            if (ok) ok = issue_g1(0);
            if (ok) ok = issue_g2(0);
            for (int it = 0; it < nit && ok; ++it) {
                if (it + 1 < nit) ok = issue_g1(it + 1);
                if (ok && it + 1 < nit) ok = issue_g2(it + 1);
            }
        }
    } else if (warp == 10) {
        // ---------------------- MMA issuer B: the dQ GEMMs ----------------------
        if (lane == 0 && nit > 0) {
            constexpr uint32_t idesc_acc = make_idesc(BF16, BT, D, false, true);
            bool ok = true;
            int ks = 0;
            uint32_t kph = 0;
            for (int it = 0; it < nit && ok; ++it) {
                ok = mbar_wait(&sm.k_full[ks], kph, status, 56);
                if (!ok) break;
                ok = mbar_wait(&sm.ds_ready, (uint32_t)it & 1u, status, 57);
                if (!ok) break;
                tc_fence_after_sync();
                const uint64_t dkm = make_sdesc(smem_u32(sm.k[ks]), PANEL, 1024);   // K as [key][channel], MN-major
                // each half of the compute threads packed its 64 keys into the first 32 of its own 64 columns
#pragma unroll
                for (int kk = 0; kk < BT / 16; ++kk)
                    umma_ts(tbase + ACC_COL, tbase + G2_COL + (kk >> 2) * 64 + (kk & 3) * 8,
                            sdesc_advance(dkm, kk * 2048), idesc_acc, it > 0 || kk > 0);
                tc_fence_before_sync();
                mbar_arrive(&sm.g2_free);           // issued, not finished: the tensor pipe runs MMAs in issue order
                umma_commit(&sm.k_empty[ks]);
                if (++ks == 3) { ks = 0; kph ^= 1u; }
            }
            umma_commit(&sm.acc_full);
        }
    } else {
        // ------------------------------ compute warps ------------------------------
        const int row_l = (warp & 3) * 32 + lane;          // query row of the tile == TMEM lane
        const int half = warp >> 2;                        // which 64 of the block's 128 keys
        const int row = r0 + row_l;
        const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);

        // Q and dO of this tile into tensor memory: this thread's row, its half of the channels,
        // as they lie in global memory (two 16-bit channels per 32-bit column).  Rows past the
        // end of Q are written as zeros.
        if (nit > 0) {
#pragma unroll
            for (int op = 0; op < 2; ++op) {
                const T *src = reinterpret_cast<const T *>(op == 0 ? q_base : do_base) +
                               (int64_t)b * (op == 0 ? q_sb : do_sb) + (int64_t)h * (op == 0 ? q_sh : do_sh) +
                               (int64_t)row * (op == 0 ? q_sn : do_sn) + half * (D / 2);
                uint32_t a[ACOLS];
#pragma unroll
                for (int i = 0; i < ACOLS; i += 4) {
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (row < p.Tq) v = __ldg(reinterpret_cast<const uint4 *>(src) + (i >> 2));
                    a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
                }
                const uint32_t dst = lane_base + (op == 0 ? QA_COL : DOA_COL) + half * ACOLS;
                if constexpr (ACOLS == 32) tmem_st32(dst, a);
                else tmem_st16(dst, a);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.a_ready);
        }
        // rows past Tq hold +inf / 0, so they yield P = 0
        const float lse_row = p.lse2[(int64_t)bh * p.Tq128 + row];
        const float dsc_row = p.delta_s[(int64_t)bh * p.Tq128 + row];
        const uint32_t scol = G1_COL + half * 64, dcol = G2_COL + half * 64;

        // P of block j from this thread's 64 scores and its row of the block's bias tile; the
        // score columns are released as soon as they are in registers
        float pv[64];
        auto load_p = [&](int j) -> bool {
            if (!mbar_wait(&sm.bb_full[j & 1], (uint32_t)(j >> 1) & 1u, status, 65)) return false;
            // 64 key columns = the whole 128-byte row of panel `half`; pv first holds
            // bias * log2(e) - lse * log2(e)
            // (vector bias: the 64 values of this half of the block, the same for every row; values past
            // the end of the keys were not loaded and are masked below)
            const unsigned char *rowp = VEC ? sm.bias[j & 1] + half * 128 : sm.bias[j & 1] + half * (BT * 128) + row_l * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                union { uint4 u; T v[8]; } cv;
                cv.u = *reinterpret_cast<const uint4 *>(rowp + (VEC ? (c << 4) : ((c ^ (row_l & 7)) << 4)));
#pragma unroll
                for (int e = 0; e < 8; ++e) pv[8 * c + e] = fmaf(to_f32<T>(cv.v[e]), LOG2E, -lse_row);
            }
            if (!mbar_wait(&sm.g1_full, (uint32_t)j & 1u, status, 60)) return false;
            tc_fence_after_sync();
            uint32_t ra[32], rb[32];
            tmem_ld32(lane_base + scol, ra);
            tmem_ld32(lane_base + scol + 32, rb);
            tmem_wait_ld();
            tc_fence_before_sync();
            mbar_arrive(&sm.s_read);
            const int blk0 = (LISTS ? (int)tl[j] : j) * BT;
            // blocks that need per-element masking: the diagonal blocks under the causal mask
            // and the block touching the end of the keys
            const bool slow = (p.causal && blk0 + BT > r0) || blk0 + BT > p.Tk;
            if (!slow) {
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    pv[i] = ex2b(fmaf(__uint_as_float(ra[i]), p.scale_log2, pv[i]));
                    pv[32 + i] = ex2b(fmaf(__uint_as_float(rb[i]), p.scale_log2, pv[32 + i]));
                }
            } else {
                const int c0 = blk0 + half * 64;
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int kj = c0 + i;
                    const bool masked = kj >= p.Tk || row >= p.Tq || (p.causal && kj > row);
                    const float sv = __uint_as_float(i < 32 ? ra[i & 31] : rb[i & 31]);
                    pv[i] = masked ? 0.f : ex2b(fmaf(sv, p.scale_log2, pv[i]));
                }
            }
            return true;
        };

        bool ok = nit > 0 ? load_p(0) : true;
        for (int it = 0; it < nit && ok; ++it) {
            // dS of block it
            ok = mbar_wait(&sm.g2_full, (uint32_t)it & 1u, status, 62);
            if (!ok) break;
            tc_fence_after_sync();
            {
                uint32_t ga[32], gb[32], pk[32];
                uint32_t qk[DBIAS ? 32 : 1];
                tmem_ld32(lane_base + dcol, ga);
                tmem_ld32(lane_base + dcol + 32, gb);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const float a0 = pv[2 * i] * fmaf(__uint_as_float(ga[2 * i]), p.scale, -dsc_row);
                    const float a1 = pv[2 * i + 1] * fmaf(__uint_as_float(ga[2 * i + 1]), p.scale, -dsc_row);
                    pk[i] = pack16b<BF16>(a0, a1);
                    const float b0 = pv[32 + 2 * i] * fmaf(__uint_as_float(gb[2 * i]), p.scale, -dsc_row);
                    const float b1 = pv[32 + 2 * i + 1] * fmaf(__uint_as_float(gb[2 * i + 1]), p.scale, -dsc_row);
                    pk[16 + i] = pack16b<BF16>(b0, b1);
                    if constexpr (DBIAS) {
                        qk[i] = pack16b<BF16>(a0 * p.inv_scale, a1 * p.inv_scale);
                        qk[16 + i] = pack16b<BF16>(b0 * p.inv_scale, b1 * p.inv_scale);
                    }
                }
                // packed dS goes to the first 32 of this thread's 64 columns, all read already
                tmem_st32(lane_base + dcol, pk);
                if constexpr (DBIAS) {
                    // bias gradient: this thread's row, the 64 keys of its half of block it
                    const int k0 = it * BT + half * 64;
                    if (row < p.Tq && k0 < p.Tk) {
                        T *dst = reinterpret_cast<T *>(p.dbias) + (int64_t)b * p.db_sb + (int64_t)h * p.db_sh +
                                 (int64_t)row * p.db_sq + k0;
                        if (p.dbias_vec && k0 + 64 <= p.Tk) {
#pragma unroll
                            for (int c = 0; c < 8; ++c)
                                __stcs(reinterpret_cast<uint4 *>(dst) + c,
                                       make_uint4(qk[4 * c], qk[4 * c + 1], qk[4 * c + 2], qk[4 * c + 3]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                union { uint32_t u; T v[2]; } cv;
                                cv.u = qk[i];
                                if (k0 + 2 * i < p.Tk) dst[2 * i] = cv.v[0];
                                if (k0 + 2 * i + 1 < p.Tk) dst[2 * i + 1] = cv.v[1];
                            }
                        }
                    }
                }
                tmem_wait_st();
            }
            tc_fence_before_sync();
            mbar_arrive(&sm.ds_ready);
            mbar_arrive(&sm.bb_empty[it & 1]);      // dS depends on every value read from the bias tile of block it
            // P of block it + 1, while the tensor pipe runs dQ(it) and dP(it + 1)
            if (it + 1 < nit) ok = load_p(it + 1);
        }

        // epilogue: dQ -> global
        if (ok && nit > 0) ok = mbar_wait(&sm.acc_full, 0, status, 63);
        tc_fence_after_sync();
        if (ok) {
            T *orow = reinterpret_cast<T *>(p.out1) + (int64_t)b * p.o1_sb + (int64_t)h * p.o1_sh + (int64_t)row * p.o1_sn;
#pragma unroll 1
            for (int c = 0; c < D / 64; ++c) {
                const int col = half * (D / 2) + c * 32;
                uint32_t r[32];
                if (nit > 0) {
                    tmem_ld32(lane_base + ACC_COL + col, r);
                    tmem_wait_ld();
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = 0u;
                }
                if (row < p.Tq) {
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

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Row statistics for the backward: delta = rowsum(O * dO)
// (flash_attn_triton_cached.py:249-292), stored pre-multiplied by the softmax
// scale, and lse * log2(e).  Rows in [Tq, Tq128) get +inf / 0 so that query
// positions past the end need no masking in the main kernels.  One warp per row.
// ---------------------------------------------------------------------------
// Rounds the fp32 dQ accumulator of the single-pass backward ([B H][16][Tq128][4], head_dim 64) into
// dQ.  One CTA per 64 queries of one (batch, head): thread = (query, 16 channels).
template <bool BF16>
__global__ void __launch_bounds__(256) attn_bwd_dq_round64_kernel(const float *__restrict__ acc, void *dq, int64_t sb, int64_t sh,
                                                                  int64_t sn, int H, int Tq, int Tq128) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int bh = blockIdx.y, b = bh / H, h = bh - b * H;
    const int q = blockIdx.x * 64 + ((int)threadIdx.x & 63), part = (int)threadIdx.x >> 6;   // channels 16 part .. + 15
    if (q >= Tq) return;
    const float4 *src = reinterpret_cast<const float4 *>(acc) + ((int64_t)bh * 16 + part * 4) * Tq128 + q;
    uint32_t w[8];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const float4 v = __ldcs(src + (int64_t)g * Tq128);        // a warp reads 512 contiguous bytes
        w[2 * g] = pack16b<BF16>(v.x, v.y);
        w[2 * g + 1] = pack16b<BF16>(v.z, v.w);
    }
    T *orow = reinterpret_cast<T *>(dq) + (int64_t)b * sb + (int64_t)h * sh + (int64_t)q * sn + part * 16;
    *reinterpret_cast<uint4 *>(orow) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4 *>(orow + 8) = make_uint4(w[4], w[5], w[6], w[7]);
}

template <typename T>
__global__ void __launch_bounds__(256) attn_bwd_prep_kernel(const __grid_constant__ AttnParams p, float *lse2, float *delta_s,
                                                            int Tq128) {
    // d / 8 lanes per row (d is 64 or 128, rows 16-byte aligned): 2 or 4 rows per warp
    const int lpr = p.d >> 3;
    const int rows_per_cta = 256 / lpr;
    const int i = blockIdx.x * rows_per_cta + (int)threadIdx.x / lpr;
    const int l = (int)threadIdx.x % lpr;
    const int bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    float a = 0.f;
    if (i < p.Tq) {
        const T *o = reinterpret_cast<const T *>(p.o) + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)i * p.o_sn;
        const T *g = reinterpret_cast<const T *>(p.d_o) + (int64_t)b * p.do_sb + (int64_t)h * p.do_sh +
                     (int64_t)i * p.do_sn;
        const Vec<T, 8> ov = load_vec_stream<T, 8>(o + l * 8), gv = load_vec<T, 8>(g + l * 8);
#pragma unroll
        for (int e = 0; e < 8; ++e) a += to_f32<T>(ov.v[e]) * to_f32<T>(gv.v[e]);
    }
    a = warp_group_sum(a, lpr);
    if (l == 0 && i < Tq128) {
        const int64_t idx = (int64_t)bh * Tq128 + i;
        delta_s[idx] = a * p.scale;
        lse2[idx] = i < p.Tq ? p.lse[(int64_t)bh * p.Tq_rounded + i] * LOG2E : INFINITY;
    }
}

// ---------------------------------------------------------------------------
// Host
// ---------------------------------------------------------------------------
int64_t tmem_bwd_workspace_bytes(int64_t B, int64_t H, int64_t Tq) {
    const int64_t Tq128 = (Tq + 127) / 128 * 128;
    return 2 * B * H * Tq128 * (int64_t)sizeof(float);
}

// The fp32 dQ accumulator of the single-pass backward (0 bytes: no such form for this head_dim); it
// follows the statistics rows in the workspace, 256-byte aligned.
int64_t single_pass_acc_offset(int64_t B, int64_t H, int64_t Tq) {
    return (tmem_bwd_workspace_bytes(B, H, Tq) + 255) / 256 * 256;
}
int64_t single_pass_acc_bytes(int64_t B, int64_t H, int64_t Tq, int64_t d) {
    if (d != 64) return 0;
    const int64_t Tq128 = (Tq + 127) / 128 * 128;
    return B * H * Tq128 * d * (int64_t)sizeof(float);
}

bool tmem_bwd_eligible(const AttnParams &p) {
    return (p.d == 64 || p.d == 128) && p.Tq >= 1 && p.Tk >= 1 && p.vec_q && p.vec_k && p.vec_v && p.vec_o && p.vec_do &&
           p.vec_dq && p.vec_dk && p.vec_dv && heads_map_encodable(p.q, p.B, p.H, p.Tq, p.q_sb, p.q_sh, p.q_sn) &&
           heads_map_encodable(p.k, p.B, p.H, p.Tk, p.k_sb, p.k_sh, p.k_sn) &&
           heads_map_encodable(p.v, p.B, p.H, p.Tk, p.v_sb, p.v_sh, p.v_sn) &&
           heads_map_encodable(p.d_o, p.B, p.H, p.Tq, p.do_sb, p.do_sh, p.do_sn);
}

template <int D, bool BF16, bool DKDV, int BIAS>
static int launch_bwd_one(const BwdTmaParams &bp, int nblocks, int BH, cudaStream_t st) {
    constexpr int BSTAGES = BIAS == 2 ? (D == 64 ? 2 : 1) : 0;
    const size_t smem = sizeof(BwdTmaSmem<D, BSTAGES>) + 1024;
    if (int e = ensure_dyn_smem(reinterpret_cast<const void *>(attn_bwd_tmem<D, BF16, DKDV, BIAS>), smem)) return e;
    dim3 grid(nblocks, BH);
    attn_bwd_tmem<D, BF16, DKDV, BIAS><<<grid, BWD_THREADS, smem, st>>>(bp);
    count_launch();
    return check_launch();
}

template <int D, bool BF16, bool DKDV>
static int launch_bwd_tmem(const BwdTmaParams &bp, int nblocks, int BH, cudaStream_t st) {
    if (bp.bias_kind != RGD_BIAS_NONE && bp.bias_vec == 2) return launch_bwd_one<D, BF16, DKDV, 2>(bp, nblocks, BH, st);
    if (bp.bias_kind != RGD_BIAS_NONE) return launch_bwd_one<D, BF16, DKDV, 1>(bp, nblocks, BH, st);
    return launch_bwd_one<D, BF16, DKDV, 0>(bp, nblocks, BH, st);
}

template <int D, bool BF16, int BIASM>
static int launch_dkdv_sub(const BwdTmaParams &bp, int nblocks, int BH, cudaStream_t st) {
    const size_t smem = sizeof(DkdvSubSmem<D, BIASM == 1 || BIASM == 3>) + 1024;
    if (int e = ensure_dyn_smem(reinterpret_cast<const void *>(attn_bwd_dkdv_sub<D, BF16, BIASM>), smem)) return e;
    dim3 grid(nblocks, BH);
    attn_bwd_dkdv_sub<D, BF16, BIASM><<<grid, DKDV_SUB_THREADS, smem, st>>>(bp);
    count_launch();
    return check_launch();
}

// Single-pass form (head_dim 64): zero the accumulator, one kernel for dK, dV and the dQ partial sums,
// round dQ.  bias_mode: 0 none, 1 matrix bias staged by TMA, 2 vector bias.
template <bool BF16>
static int bwd_single64(BwdTmaParams &bp, const AttnParams &p, int bias_mode, cudaStream_t st) {
    const int BH = p.B * p.H;
    if (cudaMemsetAsync(bp.dq_acc, 0, (size_t)BH * bp.Tq128 * 64 * sizeof(float), st) != cudaSuccess) return RGD_E_DEVICE;
    const size_t smem = (bias_mode == 1 ? sizeof(Single64Smem<true>) : sizeof(Single64Smem<false>)) + 1024;
    const void *kernel = bias_mode == 1   ? reinterpret_cast<const void *>(attn_bwd_single64<BF16, 1>)
                         : bias_mode == 2 ? reinterpret_cast<const void *>(attn_bwd_single64<BF16, 2>)
                                          : reinterpret_cast<const void *>(attn_bwd_single64<BF16, 0>);
    if (int e = ensure_dyn_smem(kernel, smem)) return e;
    dim3 grid((p.Tk + BT - 1) / BT, BH);
    if (bias_mode == 1) attn_bwd_single64<BF16, 1><<<grid, SINGLE64_THREADS, smem, st>>>(bp);
    else if (bias_mode == 2) attn_bwd_single64<BF16, 2><<<grid, SINGLE64_THREADS, smem, st>>>(bp);
    else attn_bwd_single64<BF16, 0><<<grid, SINGLE64_THREADS, smem, st>>>(bp);
    count_launch();
    if (int e = check_launch()) return e;
    dim3 rgrid((p.Tq + 63) / 64, BH);
    attn_bwd_dq_round64_kernel<BF16><<<rgrid, 256, 0, st>>>(bp.dq_acc, p.dq, p.dq_sb, p.dq_sh, p.dq_sn, p.H, p.Tq, bp.Tq128);
    count_launch();
    return check_launch();
}

template <int D, bool BF16>
static int bwd_both(BwdTmaParams &bp, const AttnParams &p, cudaStream_t st) {
    const int BH = p.B * p.H;
    bp.out1 = p.dv; bp.o1_sb = p.dv_sb; bp.o1_sh = p.dv_sh; bp.o1_sn = p.dv_sn;
    bp.out2 = p.dk; bp.o2_sb = p.dk_sb; bp.o2_sh = p.dk_sh; bp.o2_sn = p.dk_sn;
    if constexpr (D == 64) {
        // the caller gave room for the fp32 dQ accumulator: single-pass form (not with tile lists or
        // a bias gradient, which the two-kernel form serves)
        if (bp.dq_acc != nullptr && bp.dbias == nullptr && bp.tlk_cnt == nullptr && p.Tk > 0) {
            if (bp.bias_kind == RGD_BIAS_NONE) return bwd_single64<BF16>(bp, p, 0, st);
            if (bp.bias_vec == 2) return bwd_single64<BF16>(bp, p, 1, st);
            if (bp.bias_kind == RGD_BIAS_VECTOR) return bwd_single64<BF16>(bp, p, 2, st);
        }
    }
    if (bp.bias_kind == RGD_BIAS_NONE) {
        if (int e = launch_dkdv_sub<D, BF16, 0>(bp, (p.Tk + BT - 1) / BT, BH, st)) return e;
    } else if (bp.bias_vec == 2) {       // matrix bias staged by TMA, with or without tile lists
        if (bp.tlk_cnt != nullptr) {
            if (int e = launch_dkdv_sub<D, BF16, 3>(bp, (p.Tk + BT - 1) / BT, BH, st)) return e;
        } else if (int e = launch_dkdv_sub<D, BF16, 1>(bp, (p.Tk + BT - 1) / BT, BH, st)) {
            return e;
        }
    } else if (bp.bias_kind == RGD_BIAS_VECTOR) {
        if (int e = launch_dkdv_sub<D, BF16, 2>(bp, (p.Tk + BT - 1) / BT, BH, st)) return e;
    } else if (int e = launch_bwd_tmem<D, BF16, true>(bp, (p.Tk + BT - 1) / BT, BH, st)) {
        return e;
    }
    bp.out1 = p.dq; bp.o1_sb = p.dq_sb; bp.o1_sh = p.dq_sh; bp.o1_sn = p.dq_sn;
    bp.out2 = nullptr;
    if (bp.bias_kind == RGD_BIAS_VECTOR && bp.bias_vec == 1 && !bp.bias_f32 && p.Tk % 8 == 0) {
        // 16-bit vector bias, 16-byte addressable: staged per key block by one bulk copy
        const size_t smem = sizeof(DqBiasSmem<D>) + 1024;
        const void *kernel = reinterpret_cast<const void *>(attn_bwd_dq_bias<D, BF16, false, false, true>);
        if (int e = ensure_dyn_smem(kernel, smem)) return e;
        dim3 grid((p.Tq + BT - 1) / BT, BH);
        attn_bwd_dq_bias<D, BF16, false, false, true><<<grid, DQ_PIPE_THREADS, smem, st>>>(bp, p.q, p.d_o, p.q_sb, p.q_sh, p.q_sn,
                                                                                             p.do_sb, p.do_sh, p.do_sn);
        count_launch();
        return check_launch();
    }
    if (bp.bias_kind == RGD_BIAS_NONE || (bp.bias_kind == RGD_BIAS_VECTOR && bp.bias_vec != 2)) {
        const bool vec = bp.bias_kind == RGD_BIAS_VECTOR;
        const size_t smem = sizeof(DqPipeSmem<D>) + 1024;
        const void *kernel = vec ? reinterpret_cast<const void *>(attn_bwd_dq_pipe<D, BF16, true>)
                                 : reinterpret_cast<const void *>(attn_bwd_dq_pipe<D, BF16, false>);
        if (int e = ensure_dyn_smem(kernel, smem)) return e;
        dim3 grid((p.Tq + BT - 1) / BT, BH);
        if (vec) attn_bwd_dq_pipe<D, BF16, true><<<grid, DQ_PIPE_THREADS, smem, st>>>(bp);
        else attn_bwd_dq_pipe<D, BF16, false><<<grid, DQ_PIPE_THREADS, smem, st>>>(bp);
        count_launch();
        return check_launch();
    }
    if (bp.bias_vec == 2) {              // matrix bias staged by TMA
        const size_t smem = sizeof(DqBiasSmem<D>) + 1024;
        // three instantiations: plain, writing the bias gradient, following tile lists (never both)
        const int mode = bp.dbias != nullptr ? 1 : (bp.tlq_cnt != nullptr ? 2 : 0);
        const void *kernel = mode == 1   ? reinterpret_cast<const void *>(attn_bwd_dq_bias<D, BF16, true, false, false>)
                             : mode == 2 ? reinterpret_cast<const void *>(attn_bwd_dq_bias<D, BF16, false, true, false>)
                                         : reinterpret_cast<const void *>(attn_bwd_dq_bias<D, BF16, false, false, false>);
        if (int e = ensure_dyn_smem(kernel, smem)) return e;
        dim3 grid((p.Tq + BT - 1) / BT, BH);
        if (mode == 1)
            attn_bwd_dq_bias<D, BF16, true, false, false><<<grid, DQ_PIPE_THREADS, smem, st>>>(bp, p.q, p.d_o, p.q_sb, p.q_sh, p.q_sn,
                                                                                          p.do_sb, p.do_sh, p.do_sn);
        else if (mode == 2)
            attn_bwd_dq_bias<D, BF16, false, true, false><<<grid, DQ_PIPE_THREADS, smem, st>>>(bp, p.q, p.d_o, p.q_sb, p.q_sh, p.q_sn,
                                                                                          p.do_sb, p.do_sh, p.do_sn);
        else
            attn_bwd_dq_bias<D, BF16, false, false, false><<<grid, DQ_PIPE_THREADS, smem, st>>>(bp, p.q, p.d_o, p.q_sb, p.q_sh,
                                                                                           p.q_sn, p.do_sb, p.do_sh, p.do_sn);
        count_launch();
        return check_launch();
    }
    return launch_bwd_tmem<D, BF16, false>(bp, (p.Tq + BT - 1) / BT, BH, st);
}

// p.delta points at the caller's workspace (tmem_bwd_workspace_bytes); dq_acc, when not null, at an
// fp32 accumulator of single_pass_acc_bytes, which selects the single-pass form where one exists.
// Returns TMEM_NOT_TAKEN
// (nothing launched) when a descriptor cannot be encoded after all.
int tmem_bwd(const AttnParams &p, int dtype, rgd_cache *cache, float *dq_acc, cudaStream_t st) {
    BwdTmaParams bp{};
    bp.dq_acc = dq_acc;
    const bool bf16 = dtype == RGD_BF16;
    const int Tq128 = (p.Tq + 127) / 128 * 128;
    float *lse2 = p.delta, *delta_s = p.delta + (int64_t)p.B * p.H * Tq128;
    if (encode_heads_map_cached(cache, &bp.mq, p.q, p.B, p.H, p.Tq, p.d, p.q_sb, p.q_sh, p.q_sn, 64, BT, bf16) ||
        encode_heads_map_cached(cache, &bp.mk, p.k, p.B, p.H, p.Tk, p.d, p.k_sb, p.k_sh, p.k_sn, 64, BT, bf16) ||
        encode_heads_map_cached(cache, &bp.mv, p.v, p.B, p.H, p.Tk, p.d, p.v_sb, p.v_sh, p.v_sn, 64, BT, bf16) ||
        encode_heads_map_cached(cache, &bp.mdo, p.d_o, p.B, p.H, p.Tq, p.d, p.do_sb, p.do_sh, p.do_sn, 64, BT, bf16))
        return TMEM_NOT_TAKEN;
    bp.status = tmem_status_ptr();
    if (!bp.status) return RGD_E_DEVICE;
    bp.bias = p.bias; bp.b_sb = p.b_sb; bp.b_sh = p.b_sh; bp.b_sq = p.b_sq;
    bp.bias_kind = p.bias_kind; bp.bias_f32 = p.bias_f32;
    // bias_vec: 0 scalar loads, 1 rows are 16-byte addressable (vector loads), 2 staged through TMA
    bp.bias_vec = 0;
    if (p.bias_kind != RGD_BIAS_NONE && !p.bias_f32 && is_aligned(p.bias, 16) && p.b_sb % 8 == 0 && p.b_sh % 8 == 0 &&
        (p.bias_kind != RGD_BIAS_MATRIX || p.b_sq % 8 == 0))
        bp.bias_vec = 1;
    if (bias_tma_ok(p) && encode_bias_map(cache, &bp.mbias, p, bf16, BT) == RGD_OK &&
        encode_bias_map(cache, &bp.mbias64, p, bf16, 64) == RGD_OK) {
        bp.bias_vec = 2;
        bp.bias_h0 = p.b_sh == 0;
        bp.bias_b0 = p.b_sb == 0;
    }
    // The bias gradient comes out of the kernels that stage a matrix bias by TMA or take a vector
    // bias, and they recover P (dP - delta) from dS by 1 / scale; anything else: general kernels.
    if (bp.bias_vec == 2 && p.tiles != nullptr && !p.causal && p.dbias == nullptr) {
        const TileLayout L = tile_layout(bp.bias_b0 ? 1 : p.B, bp.bias_h0 ? 1 : p.H, p.Tq, p.Tk);
        bp.tlk_cnt = p.tiles + L.kcnt;
        bp.tlk_list = p.tiles + L.klist;
        bp.tlq_cnt = p.tiles + L.qcnt;
        bp.tlq_list = p.tiles + L.qlist;
        bp.tl_nqb = L.nqb;
        bp.tl_nkb = L.nkb;
    }
    bp.dbias = p.dbias; bp.db_sb = p.db_sb; bp.db_sh = p.db_sh; bp.db_sq = p.db_sq; bp.dbias_vec = p.dbias_vec;
    if (p.dbias != nullptr) {
        if (p.scale == 0.f) return TMEM_NOT_TAKEN;
        if (p.bias_kind == RGD_BIAS_MATRIX && bp.bias_vec != 2) return TMEM_NOT_TAKEN;
        if (p.bias_kind == RGD_BIAS_VECTOR && bp.bias_vec == 2) return TMEM_NOT_TAKEN;
        bp.inv_scale = 1.f / p.scale;
    }
    {
        const int rows_per_cta = 256 / (p.d / 8);
        dim3 grid((Tq128 + rows_per_cta - 1) / rows_per_cta, p.B * p.H);
        if (bf16) attn_bwd_prep_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(p, lse2, delta_s, Tq128);
        else attn_bwd_prep_kernel<__half><<<grid, 256, 0, st>>>(p, lse2, delta_s, Tq128);
        count_launch();
        if (int e = check_launch()) return e;
    }
    bp.lse2 = lse2; bp.delta_s = delta_s;
    bp.H = p.H; bp.Tq = p.Tq; bp.Tk = p.Tk; bp.Tq128 = Tq128; bp.causal = p.causal;
    bp.scale = p.scale; bp.scale_log2 = p.scale * LOG2E;
    if (p.d == 128) return bf16 ? bwd_both<128, true>(bp, p, st) : bwd_both<128, false>(bp, p, st);
    return bf16 ? bwd_both<64, true>(bp, p, st) : bwd_both<64, false>(bp, p, st);
}

}  // namespace attn
}  // namespace rgd

