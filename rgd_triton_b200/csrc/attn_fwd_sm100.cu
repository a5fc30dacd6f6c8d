// FlashAttention forward on Blackwell tensor memory (tcgen05 + TMEM + TMA).
//
// One CTA owns 256 query rows of one (batch, head) as two 128-row tiles and
// walks the keys in blocks of 128; both tiles share every K / V block, which
// is double-buffered in shared memory.  Warp roles:
//   warps 0-3  softmax of tile 0: thread r owns query row r (TMEM lane r), so
//              row maximum and row sum need no shuffles; P goes back to tensor
//              memory as packed 16-bit pairs over the S columns already read
//   warps 4-7  softmax of tile 1
//   warp 8     TMA producer: both Q tiles once, then K and V blocks (128-byte
//              swizzle, 2 stages)
//   warp 9     MMA issuer: S_t = Q_t K^T (operands in shared memory) and
//              O_t += P_t V with P read straight from tensor memory.  The issue
//              order interleaves the tiles — S of the next key block for tile 0
//              is issued between the two P V products — so one tile's softmax
//              overlaps the other tile's tensor-core work.
// Tensor memory (512 columns): S0 / P0 at 0, S1 / P1 at 128, O0 at 256, O1 at 384.
//
// Online softmax runs in the base-2 domain with a lazily updated reference
// maximum: the accumulator is only rescaled when the running maximum grows by
// more than 2^8, which keeps P <= 256 (exact in fp32, safe in 16 bits) and
// makes rescaling rare.  The result equals softmax(QK^T*scale + bias) V for any
// choice of reference, so this matches flash_attn_triton_cached.py:143-220 up
// to rounding.  Every mbarrier wait is bounded; a wait that runs out flags the
// status word, all roles drain, tensor memory is released and the host reports
// RGD_E_TIMEOUT.
#include <math.h>

#include <mutex>

#include "attn_mma.cuh"
#include "sm100_prims.cuh"

namespace rgd {
namespace attn {

using namespace rgd::sm100;

__device__ int g_tmem_status = 0;

constexpr int FWD_THREADS = 320;
constexpr int TM = 128;   // query rows per tile (two tiles per CTA)
constexpr int TN = 128;   // keys per block
constexpr float RESCALE_THRESHOLD = 8.0f;

struct FwdTmaParams {
    CUtensorMap mq, mk, mv;
    void *o;
    int64_t o_sb, o_sh, o_sn;
    const void *bias;
    int64_t b_sb, b_sh, b_sq;
    int bias_kind, bias_f32, bias_vec;
    CUtensorMap mbias;          // BIAS == 2: (Tk, Tq, H or 1, B or 1) map over the bias, box 64 x 128
    int bias_h0, bias_b0;       // bias broadcast over heads / batch: always coordinate 0
    float *lse;
    int H, Tq, Tk, Tq_rounded, causal;
    float scale_log2;   // softmax_scale * log2(e)
    int *status;        // device status word (bounded waits report here)
    // BIAS == 2, optional: per 256-query block of each bias slice, the key blocks to visit (the
    // others hold only masked bias values); null = all of them
    const uint16_t *tl_cnt, *tl_list;
    int tl_nkb;
};

// NT: query tiles per CTA.  VS: stages of V.  BS: stages of TMA-staged bias tiles per query tile
// (128 x 128, 16-bit, two 64-column panels with 128-byte swizzle; 0 = bias not staged).  With
// head_dim 128 and a staged bias everything but K is single-buffered, which is what lets both
// query tiles and their bias tiles fit: a bias tile is handed back right after the first
// softmax pass and V right after the second tile's P V product, so either reload still has most
// of an iteration to land.
// VEC: a vector bias (one value per key) is staged per key block by the softmax threads
// themselves: thread r of a tile converts the value of key r, so every thread then reads all 128
// from shared memory instead of fetching and converting them itself.
template <int D, int NT, int VS, int BS, bool VEC>
struct alignas(1024) FwdTmaSmem {
    unsigned char q[NT][TM * D * 2];
    unsigned char k[2][TN * D * 2];
    unsigned char v[VS][TN * D * 2];
    unsigned char bias[BS > 0 ? NT * BS : 1][BS > 0 ? TM * TN * 2 : 1024];
    uint64_t q_full, o_full;
    uint64_t s_full[2], p_half[2][2];           // p_half[tile][h]: P of keys [64h, 64h+64) is in tensor memory
    uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
    uint64_t b_full[2][2], b_empty[2][2];      // [tile][stage]
    uint64_t vb_ready[2];                      // [tile]: the tile's 128 threads have staged their value
    alignas(16) float vbias[VEC ? NT : 1][2][VEC ? TN : 4];   // [tile][block parity][key]: bias * log2(e)
    uint32_t tmem_base;
};

// 32 bias values (times log2 e) of tile row `row_l`, tile columns [col0, col0+32), from a
// TMA-staged tile: panel = col / 64, 16-byte chunk index XOR (row mod 8) inside the 128-byte row.
template <bool BF16>
__device__ __forceinline__ void bias_from_smem(const unsigned char *tile, int row_l, int col0, float (&b)[32]) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const unsigned char *rowp = tile + (col0 >> 6) * (TM * 128) + row_l * 128;
    const int c0 = (col0 & 63) >> 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        union { uint4 u; T v[8]; } cv;
        cv.u = *reinterpret_cast<const uint4 *>(rowp + (((c0 + i) ^ (row_l & 7)) << 4));
#pragma unroll
        for (int e = 0; e < 8; ++e) b[8 * i + e] = to_f32<T>(cv.v[e]) * LOG2E;
    }
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <bool BF16>
__device__ __forceinline__ uint32_t pack16(float a, float b) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    } else {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
}

// 32 bias values (already multiplied by log2 e) for `row`, columns [col0, col0+32).
template <bool BF16>
__device__ __forceinline__ void load_bias32(const FwdTmaParams &p, const char *bias_bh, int row, int col0, float (&b)[32]) {
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;
    const int64_t off = (p.bias_kind == RGD_BIAS_MATRIX ? (int64_t)row * p.b_sq : 0) + col0;
    const bool full = col0 + 32 <= p.Tk;
    if (p.bias_f32) {
        const float *src = reinterpret_cast<const float *>(bias_bh) + off;
        if (full && p.bias_vec) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 v = reinterpret_cast<const float4 *>(src)[i];
                b[4 * i] = v.x * LOG2E; b[4 * i + 1] = v.y * LOG2E; b[4 * i + 2] = v.z * LOG2E; b[4 * i + 3] = v.w * LOG2E;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) b[i] = (col0 + i < p.Tk) ? src[i] * LOG2E : 0.f;
        }
    } else {
        const T *src = reinterpret_cast<const T *>(bias_bh) + off;
        if (full && p.bias_vec) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const Vec<T, 8> v = load_vec<T, 8>(src + 8 * i);
#pragma unroll
                for (int e = 0; e < 8; ++e) b[8 * i + e] = to_f32<T>(v.v[e]) * LOG2E;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) b[i] = (col0 + i < p.Tk) ? to_f32<T>(src[i]) * LOG2E : 0.f;
        }
    }
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Maximum of 32 score values (three-input max: 16 instructions instead of 32).
__device__ __forceinline__ float max32(const uint32_t (&r)[32]) {
    float a = fmaxf(__uint_as_float(r[0]), __uint_as_float(r[1]));
    float b = fmaxf(__uint_as_float(r[2]), __uint_as_float(r[3]));
#pragma unroll
    for (int i = 4; i < 32; i += 4) {
        a = fmax3(a, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        b = fmax3(b, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
    }
    return fmaxf(a, b);
}

// P = 2^(s * scale_log2 - m) for 32 scores, packed to 16-bit pairs; the row sum goes to two
// accumulators so that neither addition chain is longer than 16.
template <bool BF16>
__device__ __forceinline__ void exp32(const uint32_t (&r)[32], float scale_log2, float m, uint32_t (&pk)[16], float &s0,
                                      float &s1) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float p0 = ex2(fmaf(__uint_as_float(r[i]), scale_log2, -m));
        const float p1 = ex2(fmaf(__uint_as_float(r[i + 1]), scale_log2, -m));
        const float p2 = ex2(fmaf(__uint_as_float(r[i + 2]), scale_log2, -m));
        const float p3 = ex2(fmaf(__uint_as_float(r[i + 3]), scale_log2, -m));
        s0 += p0 + p1;
        s1 += p2 + p3;
        pk[i >> 1] = pack16<BF16>(p0, p1);
        pk[(i >> 1) + 1] = pack16<BF16>(p2, p3);
    }
}

// A block with a bias that crosses the causal diagonal or the end of the keys: the two passes
// of the interior bias block of the kernel below, with x of the hidden keys set to -inf as it
// is formed.  Out of line on purpose: inlined next to the interior passes it costs those
// 8-19 % (registers), and it runs for one or two of a tile's key blocks only.  Used at
// head_dim 128 by the kernels that read the bias from global memory or a staged vector
// (BIAS == 1): in the kernels with a TMA-staged matrix bias even the call costs the interior
// blocks 4-6 % (measured at both head dims), so those keep the per-element passes at the end
// of the key loop for their masked blocks.
// `last_key`: last visible key of this thread's row, relative to the block; `bias_row`: for
// BIAS == 1 the 32-value loader's row pointer arguments, for BIAS == 2 the staged tile.
struct MaskedBiasArgs {
    uint32_t s_addr, o_addr;     // tensor-memory addresses of this thread's score and accumulator rows
    int last_key, n0, row_l, brow, j;
    const char *bias_bh;         // BIAS == 1, not staged
    const float *vbias;          // BIAS == 1, staged vector: 128 values of this block
    const unsigned char *btile;  // BIAS == 2
    float m_ref, l_sum;          // in / out
};

template <int D, bool BF16, int BIAS>
__device__ __noinline__ void masked_bias_block(const FwdTmaParams &p, MaskedBiasArgs &a, uint64_t *b_empty, uint64_t *p_half0,
                                               uint64_t *p_half1) {
    uint32_t ra[32], rb[32];
    float m0 = -INFINITY, m1 = -INFINITY;
    const uint32_t s_addr = a.s_addr;
    tmem_ld32(s_addr, ra);
    tmem_wait_ld();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        uint32_t (&cur)[32] = (c & 1) ? rb : ra;
        uint32_t (&nxt)[32] = (c & 1) ? ra : rb;
        if (c < 3) tmem_ld32(s_addr + (c + 1) * 32, nxt);
        float bb[32];
        if constexpr (BIAS == 1) {
            if (a.vbias != nullptr) {
                const float4 *src = reinterpret_cast<const float4 *>(a.vbias + c * 32);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 f = src[i];
                    bb[4 * i] = f.x; bb[4 * i + 1] = f.y; bb[4 * i + 2] = f.z; bb[4 * i + 3] = f.w;
                }
            } else {
                load_bias32<BF16>(p, a.bias_bh, a.brow, a.n0 + c * 32, bb);
            }
        }
        if constexpr (BIAS == 2) bias_from_smem<BF16>(a.btile, a.row_l, c * 32, bb);
#pragma unroll
        for (int i = 0; i < 32; ++i)
            cur[i] = (i > a.last_key - c * 32) ? 0xff800000u : __float_as_uint(fmaf(__uint_as_float(cur[i]), p.scale_log2, bb[i]));
        if (c & 1) m1 = fmaxf(m1, max32(cur));
        else m0 = fmaxf(m0, max32(cur));
        tmem_st32(s_addr + c * 32, cur);
        if (c < 3) tmem_wait_ld();
    }
    tmem_wait_st();                              // x is in tensor memory; the bias tile is consumed
    if constexpr (BIAS == 2) mbar_arrive(b_empty);
    tmem_ld32(s_addr, ra);                       // chunk 0 of x, for the second pass
    float m_ref = a.m_ref, l_sum = a.l_sum;
    const float mx = fmaxf(m0, m1);
    const bool want = (mx > m_ref + RESCALE_THRESHOLD) || (m_ref == -INFINITY && mx > -INFINITY);
    if (__any_sync(0xffffffffu, want)) {
        const float alpha = !want ? 1.f : (m_ref == -INFINITY ? 0.f : ex2(m_ref - mx));
        l_sum *= alpha;
        if (want) m_ref = mx;
        if (a.j > 0) {
            tmem_wait_ld();                      // chunk 0 of x has landed in ra; rb is free for the accumulator
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
                tmem_ld32(a.o_addr + c * 32, rb);
                tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 32; ++i) rb[i] = __float_as_uint(__uint_as_float(rb[i]) * alpha);
                tmem_st32(a.o_addr + c * 32, rb);
            }
        }
    }
    const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
    float ls0 = 0.f, ls1 = 0.f;
    uint32_t pk[16];
    tmem_wait_ld();
    tmem_ld32(s_addr + 32, rb);
    exp32<BF16>(ra, 1.0f, m_use, pk, ls0, ls1);
    tmem_st16(s_addr, pk);
    tmem_wait_ld();
    tmem_ld32(s_addr + 64, ra);
    exp32<BF16>(rb, 1.0f, m_use, pk, ls0, ls1);
    tmem_st16(s_addr + 16, pk);
    tmem_wait_ld();
    tmem_ld32(s_addr + 96, rb);
    tmem_wait_st();
    tc_fence_before_sync();
    mbar_arrive(p_half0);
    exp32<BF16>(ra, 1.0f, m_use, pk, ls0, ls1);
    tmem_st16(s_addr + 32, pk);
    tmem_wait_ld();
    exp32<BF16>(rb, 1.0f, m_use, pk, ls0, ls1);
    tmem_st16(s_addr + 48, pk);
    l_sum += ls0 + ls1;
    tmem_wait_st();
    tc_fence_before_sync();
    mbar_arrive(p_half1);
    a.m_ref = m_ref;
    a.l_sum = l_sum;
}

// BIAS: 0 none, 1 read straight from global memory by the softmax threads (vector
// bias, fp32 bias, unaligned views), 2 matrix bias staged tile by tile through TMA.
// LISTS: a matrix bias came with tile lists (an instantiation of its own: the dense form pays for
// the plumbing otherwise).
template <int D, bool BF16, int BIAS, bool LISTS>
__global__ void __launch_bounds__(FWD_THREADS, 1) attn_fwd_tmem(const __grid_constant__ FwdTmaParams p) {
    constexpr int NT = 2;
    constexpr int VS = (BIAS == 2 && D == 128) ? 1 : 2;          // stages of V
    constexpr int BS = BIAS == 2 ? (D == 128 ? 1 : 2) : 0;       // stages of bias tiles per query tile
    constexpr uint32_t BIAS_BYTES = TM * TN * 2;
    constexpr int HALVES = D / 64;                 // 64-channel (128-byte) swizzle panels per tile
    constexpr uint32_t PANEL = 128 * 64 * 2;       // bytes of one 128-row panel
    constexpr uint32_t TILE_BYTES = TM * D * 2;
    constexpr uint32_t TMEM_COLS = 512;
    using T = typename std::conditional<BF16, __nv_bfloat16, __half>::type;

    extern __shared__ unsigned char smem_raw[];
    using Smem = FwdTmaSmem<D, NT, VS, BS, BIAS == 1>;
    Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mblk = p.causal ? (int)(gridDim.x - 1 - blockIdx.x) : (int)blockIdx.x;   // heavy causal tiles first
    const int bh = blockIdx.y;
    const int b = bh / p.H, h = bh - b * p.H;
    const int m0 = mblk * NT * TM;
    // Key blocks each tile visits (a tile past the end of Q visits none; under
    // the causal mask tile 0 stops one block earlier than tile 1).
    int nb[2];
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int mt = m0 + t * TM;
        const int n_end = p.causal ? min(p.Tk, mt + TM) : p.Tk;
        nb[t] = (t < NT && mt < p.Tq) ? (n_end + TN - 1) / TN : 0;
    }
    // Key blocks to visit when the bias came with tile lists (never together with a causal mask)
    const uint16_t *tl = nullptr;
    if constexpr (LISTS) {
        const int64_t slice = (int64_t)(p.bias_b0 ? 0 : b) * (p.bias_h0 ? 1 : p.H) + (p.bias_h0 ? 0 : h);
        const int64_t idx = slice * gridDim.x + mblk;
        tl = p.tl_list + idx * p.tl_nkb;
        const int cnt = p.tl_cnt[idx];
#pragma unroll
        for (int t = 0; t < 2; ++t) nb[t] = nb[t] > 0 ? cnt : 0;
    }
    const int nblk = max(nb[0], nb[1]);
    int *status = p.status;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        mbar_init(&sm.o_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.s_full[s], 1);
            mbar_init(&sm.vb_ready[s], 128);
            mbar_init(&sm.p_half[s][0], 128);
            mbar_init(&sm.p_half[s][1], 128);
            mbar_init(&sm.k_full[s], 1);
            mbar_init(&sm.k_empty[s], 1);
            mbar_init(&sm.v_full[s], 1);
            mbar_init(&sm.v_empty[s], 1);
            for (int t = 0; t < 2; ++t) {
                mbar_init(&sm.b_full[t][s], 1);
                mbar_init(&sm.b_empty[t][s], 128);
            }
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
        if (lane == 0) {
            tma_prefetch_desc(&p.mq);
            tma_prefetch_desc(&p.mk);
            tma_prefetch_desc(&p.mv);
            if constexpr (BIAS == 2) tma_prefetch_desc(&p.mbias);
            mbar_expect_tx(&sm.q_full, NT * TILE_BYTES);
            for (int t = 0; t < NT; ++t)
                for (int hh = 0; hh < HALVES; ++hh)
                    tma_load_4d(sm.q[t] + hh * PANEL, &p.mq, &sm.q_full, hh * 64, m0 + t * TM, h, b);
            bool ok = true;
            for (int j = 0; j < nblk; ++j) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u;
                ok = mbar_wait(&sm.k_empty[s], ph ^ 1u, status, 11);
                if (!ok) break;
                mbar_expect_tx(&sm.k_full[s], TILE_BYTES);
                for (int hh = 0; hh < HALVES; ++hh)
                    tma_load_4d(sm.k[s] + hh * PANEL, &p.mk, &sm.k_full[s], hh * 64, (LISTS ? (int)tl[j] : j) * TN, h, b);
                if constexpr (BIAS == 2) {
                    const int bs = j % BS;
                    const uint32_t bph = (uint32_t)(j / BS) & 1u;
                    for (int t = 0; t < NT && ok; ++t) {
                        if (j >= nb[t]) continue;
                        ok = mbar_wait(&sm.b_empty[t][bs], bph ^ 1u, status, 13);
                        if (!ok) break;
                        mbar_expect_tx(&sm.b_full[t][bs], BIAS_BYTES);
                        for (int pn = 0; pn < 2; ++pn)
                            tma_load_4d(sm.bias[t * BS + bs] + pn * (TM * 128), &p.mbias, &sm.b_full[t][bs],
                                        (LISTS ? (int)tl[j] : j) * TN + pn * 64, m0 + t * TM, p.bias_h0 ? 0 : h, p.bias_b0 ? 0 : b);
                    }
                    if (!ok) break;
                }
                const int vs = j % VS;
                ok = mbar_wait(&sm.v_empty[vs], ((uint32_t)(j / VS) & 1u) ^ 1u, status, 12);
                if (!ok) break;
                mbar_expect_tx(&sm.v_full[vs], TILE_BYTES);
                for (int hh = 0; hh < HALVES; ++hh)
                    tma_load_4d(sm.v[vs] + hh * PANEL, &p.mv, &sm.v_full[vs], hh * 64, (LISTS ? (int)tl[j] : j) * TN, h, b);
            }
            if (!ok) {
                // Give copies already in flight time to land before the CTA goes away.
                for (int i = 0; i < 64; ++i) __nanosleep(1000);
            }
        }
    } else if (warp == 9) {
        // ------------------------------ MMA issuer ------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = make_idesc(BF16, TM, TN, false, false);
            constexpr uint32_t idesc_pv = make_idesc(BF16, TM, D, false, true);
            auto issue_s = [&](int t, int s) {
                const uint32_t q_addr = smem_u32(sm.q[t]), k_addr = smem_u32(sm.k[s]);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = (kk / 4) * PANEL + (kk % 4) * 32;
                    umma_ss(tbase + t * 128, make_sdesc(q_addr + off, 16, 1024), make_sdesc(k_addr + off, 16, 1024),
                            idesc_qk, kk > 0);
                }
                umma_commit(&sm.s_full[t]);
            };
            // O_t += P_t[:, 64h .. 64h+64) V[64h .. 64h+64, :]: the first half can run while the
            // softmax threads still form the second half of P
            auto issue_pv = [&](int t, int s, int h, bool first) {
                const uint32_t v_addr = smem_u32(sm.v[s]);
#pragma unroll
                for (int kk = 4 * h; kk < 4 * h + 4; ++kk)
                    umma_ts(tbase + 256 + t * 128, tbase + t * 128 + kk * 8, make_sdesc(v_addr + kk * 2048, PANEL, 1024),
                            idesc_pv, !first || kk > 0);
            };
            bool ok = nblk > 0 ? mbar_wait(&sm.q_full, 0, status, 21) : true;
            if (ok && nblk > 0) ok = mbar_wait(&sm.k_full[0], 0, status, 22);
            if (ok && nblk > 0) {
                tc_fence_after_sync();
                if (nb[0] > 0) issue_s(0, 0);
                if (nb[1] > 0) issue_s(1, 0);
                umma_commit(&sm.k_empty[0]);
            }
            for (int j = 0; j < nblk && ok; ++j) {
                const int s = j & 1;
                const uint32_t ph = (uint32_t)(j >> 1) & 1u, par = (uint32_t)j & 1u;
                const bool more = j + 1 < nblk;
                const int vs = j % VS;
                ok = mbar_wait(&sm.v_full[vs], (uint32_t)(j / VS) & 1u, status, 23);
                if (!ok) break;
                if (j < nb[0]) {
                    ok = mbar_wait(&sm.p_half[0][0], par, status, 24);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv(0, vs, 0, j == 0);
                    ok = mbar_wait(&sm.p_half[0][1], par, status, 27);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv(0, vs, 1, false);
                }
                if (more) {
                    ok = mbar_wait(&sm.k_full[s ^ 1], (uint32_t)((j + 1) >> 1) & 1u, status, 25);
                    if (!ok) break;
                    tc_fence_after_sync();
                    if (j + 1 < nb[0]) issue_s(0, s ^ 1);
                }
                if (j < nb[1]) {
                    ok = mbar_wait(&sm.p_half[1][0], par, status, 26);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv(1, vs, 0, j == 0);
                    ok = mbar_wait(&sm.p_half[1][1], par, status, 28);
                    if (!ok) break;
                    tc_fence_after_sync();
                    issue_pv(1, vs, 1, false);
                }
                umma_commit(&sm.v_empty[vs]);
                if (more) {
                    if (j + 1 < nb[1]) issue_s(1, s ^ 1);
                    umma_commit(&sm.k_empty[s ^ 1]);
                }
            }
            umma_commit(&sm.o_full);
        }
    } else {
        // ------------------------------ softmax + epilogue ------------------------------
        const int t = warp >> 2;                         // which query tile
        const int row_l = (warp & 3) * 32 + lane;        // row inside the tile == TMEM lane
        const int row = m0 + t * TM + row_l;
        const uint32_t lane_base = tbase + ((uint32_t)((warp & 3) * 32) << 16);
        const uint32_t s_col = t * 128, o_col = 256 + t * 128;
        const int my_nb = nb[t];
        const char *bias_bh = nullptr;
        if constexpr (BIAS == 1)
            bias_bh = reinterpret_cast<const char *>(p.bias) +
                      ((int64_t)b * p.b_sb + (int64_t)h * p.b_sh) * (p.bias_f32 ? 4 : 2);
        const int brow = row < p.Tq ? row : (p.Tq - 1);     // rows past the end read a valid bias row

        const bool vec_staged = BIAS == 1 && p.bias_kind == RGD_BIAS_VECTOR;
        float m_ref = -INFINITY, l_sum = 0.f;
        bool ok = true;
        for (int j = 0; j < my_nb; ++j) {
            if constexpr (BIAS == 1) {
                if (vec_staged) {
                    // this thread's key of the block: one value, times log2(e), for the whole tile
                    const int kj = j * TN + row_l;
                    float bvl = 0.f;
                    if (kj < p.Tk)
                        bvl = p.bias_f32 ? reinterpret_cast<const float *>(bias_bh)[kj]
                                         : to_f32<T>(reinterpret_cast<const T *>(bias_bh)[kj]);
                    sm.vbias[t][j & 1][row_l] = bvl * LOG2E;
                    mbar_arrive(&sm.vb_ready[t]);
                }
            }
            ok = mbar_wait(&sm.s_full[t], (uint32_t)j & 1u, status, 31);
            if (!ok) break;
            if constexpr (BIAS == 1) {
                if (vec_staged) {
                    ok = mbar_wait(&sm.vb_ready[t], (uint32_t)j & 1u, status, 34);
                    if (!ok) break;
                }
            }
            tc_fence_after_sync();
            const unsigned char *btile = nullptr;
            constexpr int BSD = BS > 0 ? BS : 1;
            if constexpr (BIAS == 2) {
                ok = mbar_wait(&sm.b_full[t][j % BSD], (uint32_t)(j / BSD) & 1u, status, 33);
                if (!ok) break;
                btile = sm.bias[t * BSD + (j % BSD)];
            }
            const int n0 = (LISTS ? (int)tl[j] : j) * TN;
            const bool need_mask = (n0 + TN > p.Tk) || (p.causal && n0 + TN > m0 + t * TM);

            const uint32_t s_addr = lane_base + s_col;
            if (BIAS == 0 && !need_mask) {
                // ---- interior block, no bias: the loads of tensor memory run one 32-column chunk
                // ahead of the arithmetic in both passes, so their latency is paid once per block
                // and not once per chunk; P leaves in two halves, so the first P V product
                // starts while the second half's exponentials are still being taken ----
                uint32_t ra[32], rb[32];
                tmem_ld32(s_addr, ra);
                tmem_wait_ld();
                tmem_ld32(s_addr + 32, rb);
                float m0 = max32(ra);
                tmem_wait_ld();
                tmem_ld32(s_addr + 64, ra);
                float m1 = max32(rb);
                tmem_wait_ld();
                tmem_ld32(s_addr + 96, rb);
                m0 = fmaxf(m0, max32(ra));
                tmem_wait_ld();
                tmem_ld32(s_addr, ra);                       // chunk 0 again, for the second pass
                m1 = fmaxf(m1, max32(rb));
                const float mx = fmaxf(m0, m1) * p.scale_log2;          // scale > 0: max commutes with it
                const bool want = (mx > m_ref + RESCALE_THRESHOLD) || (m_ref == -INFINITY && mx > -INFINITY);
                if (__any_sync(0xffffffffu, want)) {
                    const float alpha = !want ? 1.f : (m_ref == -INFINITY ? 0.f : ex2(m_ref - mx));
                    l_sum *= alpha;
                    if (want) m_ref = mx;
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t r[32];
                            tmem_ld32(lane_base + o_col + c * 32, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                            tmem_st32(lane_base + o_col + c * 32, r);
                        }
                    }
                }
                const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
                float ls0 = 0.f, ls1 = 0.f;
                uint32_t pk[16];
                tmem_wait_ld();
                tmem_ld32(s_addr + 32, rb);
                exp32<BF16>(ra, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr, pk);                       // packed P over columns already read
                tmem_wait_ld();
                tmem_ld32(s_addr + 64, ra);
                exp32<BF16>(rb, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 16, pk);
                tmem_wait_ld();
                tmem_ld32(s_addr + 96, rb);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.p_half[t][0]);               // keys 0..63 of P are in place
                exp32<BF16>(ra, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 32, pk);
                tmem_wait_ld();
                exp32<BF16>(rb, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 48, pk);
                l_sum += ls0 + ls1;
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.p_half[t][1]);
                continue;
            }

            if (BIAS == 0 && need_mask) {
                // ---- no bias, block crossing the causal diagonal or the end of the keys: the
                // same pipelined passes as above (a copy of their own, so that the interior blocks'
                // code stays as it is), with the hidden scores set to -inf in registers as each
                // chunk arrives.  Every row of a visited block keeps at least its first key, so
                // the block maximum stays finite. ----
                const int last_key = min(p.Tk - 1, p.causal ? row : p.Tk - 1) - n0;   // last visible key of this row, block-relative
                auto mask32 = [&](uint32_t (&r)[32], int c0) {
                    const int lim = last_key - c0;
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (i > lim) r[i] = 0xff800000u;          // -inf
                };
                uint32_t ra[32], rb[32];
                tmem_ld32(s_addr, ra);
                tmem_wait_ld();
                tmem_ld32(s_addr + 32, rb);
                mask32(ra, 0);
                float m0 = max32(ra);
                tmem_wait_ld();
                tmem_ld32(s_addr + 64, ra);
                mask32(rb, 32);
                float m1 = max32(rb);
                tmem_wait_ld();
                tmem_ld32(s_addr + 96, rb);
                mask32(ra, 64);
                m0 = fmaxf(m0, max32(ra));
                tmem_wait_ld();
                tmem_ld32(s_addr, ra);                       // chunk 0 again, for the second pass
                mask32(rb, 96);
                m1 = fmaxf(m1, max32(rb));
                const float mx = fmaxf(m0, m1) * p.scale_log2;          // scale > 0: max commutes with it
                const bool want = (mx > m_ref + RESCALE_THRESHOLD) || (m_ref == -INFINITY && mx > -INFINITY);
                if (__any_sync(0xffffffffu, want)) {
                    const float alpha = !want ? 1.f : (m_ref == -INFINITY ? 0.f : ex2(m_ref - mx));
                    l_sum *= alpha;
                    if (want) m_ref = mx;
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t r[32];
                            tmem_ld32(lane_base + o_col + c * 32, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                            tmem_st32(lane_base + o_col + c * 32, r);
                        }
                    }
                }
                const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
                float ls0 = 0.f, ls1 = 0.f;
                uint32_t pk[16];
                tmem_wait_ld();
                tmem_ld32(s_addr + 32, rb);
                mask32(ra, 0);
                exp32<BF16>(ra, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr, pk);                       // packed P over columns already read
                tmem_wait_ld();
                tmem_ld32(s_addr + 64, ra);
                mask32(rb, 32);
                exp32<BF16>(rb, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 16, pk);
                tmem_wait_ld();
                tmem_ld32(s_addr + 96, rb);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.p_half[t][0]);               // keys 0..63 of P are in place
                mask32(ra, 64);
                exp32<BF16>(ra, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 32, pk);
                tmem_wait_ld();
                mask32(rb, 96);
                exp32<BF16>(rb, p.scale_log2, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 48, pk);
                l_sum += ls0 + ls1;
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.p_half[t][1]);
                continue;
            }

            if (BIAS != 0 && !need_mask) {
                // ---- interior block with a bias: x = s * scale * log2e + bias * log2e is formed
                // ONCE per element (the bias tile is read and converted once), written back over
                // the score columns and reduced to the row maximum in the same pass; the second
                // pass is the one of the no-bias path, on x.  Loads run one chunk ahead. ----
                uint32_t ra[32], rb[32];
                float m0 = -INFINITY, m1 = -INFINITY;
                tmem_ld32(s_addr, ra);
                tmem_wait_ld();
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t (&cur)[32] = (c & 1) ? rb : ra;
                    uint32_t (&nxt)[32] = (c & 1) ? ra : rb;
                    if (c < 3) tmem_ld32(s_addr + (c + 1) * 32, nxt);
                    float bb[32];
                    if constexpr (BIAS == 1) {
                        if (vec_staged) {
                            const float4 *src = reinterpret_cast<const float4 *>(&sm.vbias[BIAS == 1 ? t : 0][j & 1][c * 32]);
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const float4 f = src[i];
                                bb[4 * i] = f.x; bb[4 * i + 1] = f.y; bb[4 * i + 2] = f.z; bb[4 * i + 3] = f.w;
                            }
                        } else {
                            load_bias32<BF16>(p, bias_bh, brow, n0 + c * 32, bb);
                        }
                    }
                    if constexpr (BIAS == 2) bias_from_smem<BF16>(btile, row_l, c * 32, bb);
#pragma unroll
                    for (int i = 0; i < 32; ++i) cur[i] = __float_as_uint(fmaf(__uint_as_float(cur[i]), p.scale_log2, bb[i]));
                    if (c & 1) m1 = fmaxf(m1, max32(cur));
                    else m0 = fmaxf(m0, max32(cur));
                    tmem_st32(s_addr + c * 32, cur);
                    if (c < 3) tmem_wait_ld();
                }
                tmem_wait_st();                              // x is in tensor memory; the bias tile is consumed
                if constexpr (BIAS == 2) mbar_arrive(&sm.b_empty[t][j % BSD]);
                tmem_ld32(s_addr, ra);                       // chunk 0 of x, for the second pass
                const float mx = fmaxf(m0, m1);
                const bool want = (mx > m_ref + RESCALE_THRESHOLD) || (m_ref == -INFINITY && mx > -INFINITY);
                if (__any_sync(0xffffffffu, want)) {
                    const float alpha = !want ? 1.f : (m_ref == -INFINITY ? 0.f : ex2(m_ref - mx));
                    l_sum *= alpha;
                    if (want) m_ref = mx;
                    if (j > 0) {
#pragma unroll 1
                        for (int c = 0; c < D / 32; ++c) {
                            uint32_t r[32];
                            tmem_ld32(lane_base + o_col + c * 32, r);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                            tmem_st32(lane_base + o_col + c * 32, r);
                        }
                    }
                }
                const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
                float ls0 = 0.f, ls1 = 0.f;
                uint32_t pk[16];
                tmem_wait_ld();
                tmem_ld32(s_addr + 32, rb);
                exp32<BF16>(ra, 1.0f, m_use, pk, ls0, ls1);
                tmem_st16(s_addr, pk);
                tmem_wait_ld();
                tmem_ld32(s_addr + 64, ra);
                exp32<BF16>(rb, 1.0f, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 16, pk);
                tmem_wait_ld();
                tmem_ld32(s_addr + 96, rb);
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.p_half[t][0]);
                exp32<BF16>(ra, 1.0f, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 32, pk);
                tmem_wait_ld();
                exp32<BF16>(rb, 1.0f, m_use, pk, ls0, ls1);
                tmem_st16(s_addr + 48, pk);
                l_sum += ls0 + ls1;
                tmem_wait_st();
                tc_fence_before_sync();
                mbar_arrive(&sm.p_half[t][1]);
                continue;
            }

            if constexpr (BIAS == 1 && D == 128) {
                // a block with a bias that crosses the causal diagonal or the end of the keys
                MaskedBiasArgs a;
                a.s_addr = s_addr;
                a.o_addr = lane_base + o_col;
                a.last_key = min(p.Tk - 1, p.causal ? row : p.Tk - 1) - n0;
                a.n0 = n0;
                a.row_l = row_l;
                a.brow = brow;
                a.j = j;
                a.bias_bh = bias_bh;
                a.vbias = (BIAS == 1 && vec_staged) ? &sm.vbias[BIAS == 1 ? t : 0][j & 1][0] : nullptr;
                a.btile = btile;
                a.m_ref = m_ref;
                a.l_sum = l_sum;
                masked_bias_block<D, BF16, BIAS>(p, a, BIAS == 2 ? &sm.b_empty[t][j % BSD] : nullptr, &sm.p_half[t][0],
                                                 &sm.p_half[t][1]);
                m_ref = a.m_ref;
                l_sum = a.l_sum;
                continue;
            }

            // pass 1: block maximum of x = s * scale * log2e + bias * log2e, 64 columns per round
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t r0[32], r1[32];
                tmem_ld32(lane_base + s_col + c * 64, r0);
                tmem_ld32(lane_base + s_col + c * 64 + 32, r1);
                if (BIAS == 0 && !need_mask) {
                    tmem_wait_ld();
                    float a = -INFINITY, bq = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        a = fmaxf(a, __uint_as_float(r0[i]));
                        bq = fmaxf(bq, __uint_as_float(r1[i]));
                    }
                    mx = fmaxf(mx, fmaxf(a, bq) * p.scale_log2);      // scale > 0: max commutes with it
                } else {
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        float bb[32];
                        if constexpr (BIAS == 1) load_bias32<BF16>(p, bias_bh, brow, n0 + c * 64 + hf * 32, bb);
                        if constexpr (BIAS == 2) bias_from_smem<BF16>(btile, row_l, c * 64 + hf * 32, bb);
                        if (hf == 0) tmem_wait_ld();
                        // two copies of the loop, so that blocks without a mask carry no per-element test
                        if (need_mask) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                float x = __uint_as_float(hf ? r1[i] : r0[i]) * p.scale_log2;
                                if constexpr (BIAS != 0) x += bb[i];
                                const int col = n0 + c * 64 + hf * 32 + i;
                                if (col >= p.Tk || (p.causal && col > row)) x = -INFINITY;
                                mx = fmaxf(mx, x);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                float x = __uint_as_float(hf ? r1[i] : r0[i]) * p.scale_log2;
                                if constexpr (BIAS != 0) x += bb[i];
                                mx = fmaxf(mx, x);
                            }
                        }
                    }
                }
            }
            // lazy reference update (warp-uniform decision: TMEM accesses are warp-collective)
            const bool want = (mx > m_ref + RESCALE_THRESHOLD) || (m_ref == -INFINITY && mx > -INFINITY);
            if (__any_sync(0xffffffffu, want)) {
                // lanes that keep their reference scale by exactly 1
                const float alpha = !want ? 1.f : (m_ref == -INFINITY ? 0.f : ex2(m_ref - mx));
                l_sum *= alpha;
                if (want) m_ref = mx;
                if (j > 0) {
#pragma unroll 1
                    for (int c = 0; c < D / 32; ++c) {
                        uint32_t r[32];
                        tmem_ld32(lane_base + o_col + c * 32, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_st32(lane_base + o_col + c * 32, r);
                    }
                }
            }
            const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;

            // pass 2: P = 2^(x - m), row sum, packed 16-bit P over the consumed S columns
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                uint32_t r0[32], r1[32];
                tmem_ld32(lane_base + s_col + c * 64, r0);
                tmem_ld32(lane_base + s_col + c * 64 + 32, r1);
                uint32_t pk[32];
                float ls0 = 0.f, ls1 = 0.f;
                if (BIAS == 0 && !need_mask) {
                    tmem_wait_ld();
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2(fmaf(__uint_as_float(r0[i]), p.scale_log2, -m_use));
                        const float p1 = ex2(fmaf(__uint_as_float(r0[i + 1]), p.scale_log2, -m_use));
                        const float p2 = ex2(fmaf(__uint_as_float(r1[i]), p.scale_log2, -m_use));
                        const float p3 = ex2(fmaf(__uint_as_float(r1[i + 1]), p.scale_log2, -m_use));
                        ls0 += p0 + p1;
                        ls1 += p2 + p3;
                        pk[i >> 1] = pack16<BF16>(p0, p1);
                        pk[16 + (i >> 1)] = pack16<BF16>(p2, p3);
                    }
                } else {
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        float bb[32];
                        if constexpr (BIAS == 1) load_bias32<BF16>(p, bias_bh, brow, n0 + c * 64 + hf * 32, bb);
                        if constexpr (BIAS == 2) bias_from_smem<BF16>(btile, row_l, c * 64 + hf * 32, bb);
                        if (hf == 0) tmem_wait_ld();
                        if (need_mask) {
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                float x0 = __uint_as_float(hf ? r1[i] : r0[i]) * p.scale_log2;
                                float x1 = __uint_as_float(hf ? r1[i + 1] : r0[i + 1]) * p.scale_log2;
                                if constexpr (BIAS != 0) {
                                    x0 += bb[i];
                                    x1 += bb[i + 1];
                                }
                                const int col = n0 + c * 64 + hf * 32 + i;
                                if (col >= p.Tk || (p.causal && col > row)) x0 = -INFINITY;
                                if (col + 1 >= p.Tk || (p.causal && col + 1 > row)) x1 = -INFINITY;
                                const float p0 = ex2(x0 - m_use), p1 = ex2(x1 - m_use);
                                ls0 += p0 + p1;
                                pk[hf * 16 + (i >> 1)] = pack16<BF16>(p0, p1);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                float x0 = __uint_as_float(hf ? r1[i] : r0[i]) * p.scale_log2;
                                float x1 = __uint_as_float(hf ? r1[i + 1] : r0[i + 1]) * p.scale_log2;
                                if constexpr (BIAS != 0) {
                                    x0 += bb[i];
                                    x1 += bb[i + 1];
                                }
                                const float p0 = ex2(x0 - m_use), p1 = ex2(x1 - m_use);
                                ls0 += p0 + p1;
                                pk[hf * 16 + (i >> 1)] = pack16<BF16>(p0, p1);
                            }
                        }
                    }
                }
                l_sum += ls0 + ls1;
                tmem_st32(lane_base + s_col + c * 32, pk);
            }
            tmem_wait_st();
            tc_fence_before_sync();
            mbar_arrive(&sm.p_half[t][0]);
            mbar_arrive(&sm.p_half[t][1]);
            if constexpr (BIAS == 2) mbar_arrive(&sm.b_empty[t][j % BSD]);   // bias tile read twice, now free
        }

        // epilogue: O / l, LSE
        if (my_nb > 0) {
            if (ok) ok = mbar_wait(&sm.o_full, 0, status, 32);
            tc_fence_after_sync();
            const float inv = l_sum > 0.f ? 1.0f / l_sum : 0.f;
            if (ok) {
                T *orow = reinterpret_cast<T *>(p.o) + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)row * p.o_sn;
#pragma unroll 1
                for (int c = 0; c < D / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(lane_base + o_col + c * 32, r);
                    tmem_wait_ld();
                    if (row < p.Tq) {
#pragma unroll
                        for (int i = 0; i < 32; i += 8) {
                            uint4 v;
                            v.x = pack16<BF16>(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
                            v.y = pack16<BF16>(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
                            v.z = pack16<BF16>(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
                            v.w = pack16<BF16>(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
                            *reinterpret_cast<uint4 *>(orow + c * 32 + i) = v;
                        }
                    }
                }
                if (row < p.Tq_rounded) {
                    const float lse = l_sum > 0.f ? (m_ref + log2f(l_sum)) * 0.6931471805599453f : -INFINITY;
                    p.lse[(int64_t)bh * p.Tq_rounded + row] = row < p.Tq ? lse : INFINITY;
                }
            }
        } else if (row < p.Tq_rounded) {
            // tile entirely past the end of Q: only the padded LSE rows exist
            p.lse[(int64_t)bh * p.Tq_rounded + row] = INFINITY;
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, TMEM_COLS);
}

// ---------------------------------------------------------------------------
// Host
// ---------------------------------------------------------------------------
// Device address of the status word on the current device (the symbol has one
// instance per device, so the address is looked up per device and cached).
int *tmem_status_ptr() {
    static std::mutex mu;
    static int *cache[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (cache[dev] == nullptr) {
        void *ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_tmem_status) != cudaSuccess) {
            (void)cudaGetLastError();
            return nullptr;
        }
        cache[dev] = reinterpret_cast<int *>(ptr);
    }
    return cache[dev];
}

// Views the TMA descriptors can describe: 16-byte addressable rows, and for every dimension
// of extent > 1 a positive stride (a tensor expanded over batch or heads has stride 0 there
// and takes the general kernels).
static bool tma_view_ok(const void *ptr, int B, int H, int T, int64_t sb, int64_t sh, int64_t sn) {
    return heads_map_encodable(ptr, B, H, T, sb, sh, sn);
}

bool tmem_fwd_eligible(const AttnParams &p) {
    // The mask-free fast path takes the block maximum before scaling, which needs scale > 0.
    return (p.d == 64 || p.d == 128) && p.Tq >= 1 && p.Tk >= 1 && p.scale > 0.f && p.vec_q && p.vec_k && p.vec_v &&
           p.vec_o && tma_view_ok(p.q, p.B, p.H, p.Tq, p.q_sb, p.q_sh, p.q_sn) &&
           tma_view_ok(p.k, p.B, p.H, p.Tk, p.k_sb, p.k_sh, p.k_sn) &&
           tma_view_ok(p.v, p.B, p.H, p.Tk, p.v_sb, p.v_sh, p.v_sn);
}

template <int D, bool BF16, int BIAS, bool LISTS = false>
static int launch_fwd_one(const FwdTmaParams &fp, int Tq, int BH, cudaStream_t st) {
    constexpr int NT = 2;
    constexpr int VS = (BIAS == 2 && D == 128) ? 1 : 2;
    constexpr int BS = BIAS == 2 ? (D == 128 ? 1 : 2) : 0;
    const size_t smem = sizeof(FwdTmaSmem<D, NT, VS, BS, BIAS == 1>) + 1024;
    if (int e = ensure_dyn_smem(reinterpret_cast<const void *>(attn_fwd_tmem<D, BF16, BIAS, LISTS>), smem)) return e;
    dim3 grid((Tq + NT * TM - 1) / (NT * TM), BH);
    attn_fwd_tmem<D, BF16, BIAS, LISTS><<<grid, FWD_THREADS, smem, st>>>(fp);
    count_launch();
    return check_launch();
}

template <int D, bool BF16>
static int launch_fwd_tmem(const FwdTmaParams &fp, int bias_mode, int Tq, int BH, cudaStream_t st) {
    if (bias_mode == 2 && fp.tl_cnt != nullptr) return launch_fwd_one<D, BF16, 2, true>(fp, Tq, BH, st);
    if (bias_mode == 2) return launch_fwd_one<D, BF16, 2>(fp, Tq, BH, st);
    if (bias_mode == 1) return launch_fwd_one<D, BF16, 1>(fp, Tq, BH, st);
    return launch_fwd_one<D, BF16, 0>(fp, Tq, BH, st);
}

// A matrix bias in the tensor dtype whose rows are 16-byte addressable goes through TMA.
bool bias_tma_ok(const AttnParams &p) {
    if (p.bias_kind != RGD_BIAS_MATRIX || p.bias_f32) return false;
    if (!is_aligned(p.bias, 16) || p.b_sq % 8 != 0 || p.b_sq <= 0 || p.Tk % 8 != 0) return false;
    if (p.b_sh % 8 != 0 || p.b_sb % 8 != 0 || p.b_sh < 0 || p.b_sb < 0) return false;
    return true;
}

// (Tk, Tq, H or 1, B or 1) map over the bias; broadcast dims (stride 0) become extent 1.
int encode_bias_map(rgd_cache *cache, CUtensorMap *out, const AttnParams &p, bool bf16, int box_q) {
    const int64_t Hb = p.b_sh == 0 ? 1 : p.H, Bb = p.b_sb == 0 ? 1 : p.B;
    return encode_heads_map_cached(cache, out, p.bias, Bb, Hb, p.Tq, p.Tk, p.b_sb, p.b_sh, p.b_sq, 64, box_q, bf16);
}

// Returns TMEM_NOT_TAKEN (nothing launched) when a descriptor cannot be encoded after all; the
// caller then runs the general kernels.
int tmem_fwd(const AttnParams &p, int dtype, rgd_cache *cache, cudaStream_t st) {
    FwdTmaParams fp{};
    const bool bf16 = dtype == RGD_BF16;
    if (encode_heads_map_cached(cache, &fp.mq, p.q, p.B, p.H, p.Tq, p.d, p.q_sb, p.q_sh, p.q_sn, 64, TM, bf16) ||
        encode_heads_map_cached(cache, &fp.mk, p.k, p.B, p.H, p.Tk, p.d, p.k_sb, p.k_sh, p.k_sn, 64, TN, bf16) ||
        encode_heads_map_cached(cache, &fp.mv, p.v, p.B, p.H, p.Tk, p.d, p.v_sb, p.v_sh, p.v_sn, 64, TN, bf16))
        return TMEM_NOT_TAKEN;
    fp.o = p.out_o; fp.o_sb = p.o_sb; fp.o_sh = p.o_sh; fp.o_sn = p.o_sn;
    fp.bias = p.bias; fp.b_sb = p.b_sb; fp.b_sh = p.b_sh; fp.b_sq = p.b_sq;
    fp.bias_kind = p.bias_kind; fp.bias_f32 = p.bias_f32;
    const int bel = p.bias_f32 ? 4 : 8;   // bias elements per 16 bytes
    fp.bias_vec = p.bias_kind != RGD_BIAS_NONE && is_aligned(p.bias, 16) && p.b_sb % bel == 0 && p.b_sh % bel == 0 &&
                  (p.bias_kind != RGD_BIAS_MATRIX || p.b_sq % bel == 0);
    int bias_mode = p.bias_kind == RGD_BIAS_NONE ? 0 : 1;
    if (bias_mode == 1 && bias_tma_ok(p) && encode_bias_map(cache, &fp.mbias, p, bf16, TM) == RGD_OK) {
        bias_mode = 2;
        fp.bias_h0 = p.b_sh == 0;
        fp.bias_b0 = p.b_sb == 0;
    }
    if (bias_mode == 2 && p.tiles != nullptr && !p.causal) {
        const TileLayout L = tile_layout(fp.bias_b0 ? 1 : p.B, fp.bias_h0 ? 1 : p.H, p.Tq, p.Tk);
        fp.tl_cnt = p.tiles + L.q2cnt;
        fp.tl_list = p.tiles + L.q2list;
        fp.tl_nkb = L.nkb;
    }
    fp.lse = p.lse;
    fp.H = p.H; fp.Tq = p.Tq; fp.Tk = p.Tk; fp.Tq_rounded = p.Tq_rounded; fp.causal = p.causal;
    fp.scale_log2 = p.scale * LOG2E;
    fp.status = tmem_status_ptr();
    if (!fp.status) return RGD_E_DEVICE;
    const int BH = p.B * p.H;
    if (p.d == 128)
        return bf16 ? launch_fwd_tmem<128, true>(fp, bias_mode, p.Tq, BH, st) : launch_fwd_tmem<128, false>(fp, bias_mode, p.Tq, BH, st);
    return bf16 ? launch_fwd_tmem<64, true>(fp, bias_mode, p.Tq, BH, st) : launch_fwd_tmem<64, false>(fp, bias_mode, p.Tq, BH, st);
}

// Exercises the give-up path of the bounded waits without any broken pipeline: one thread waits,
// with a short limit, on an mbarrier that nothing ever arrives at.  The wait runs out, records
// its site code in the status word and the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(int *status, unsigned long long limit_ns, int *gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        fence_mbar_init();
        const bool completed = mbar_wait(&bar, 0, status, 99, limit_ns);
        if (gave_up) *gave_up = completed ? 0 : 1;
    }
}

int bounded_wait_selftest(int64_t limit_ns, cudaStream_t st) {
    int *status = tmem_status_ptr();
    if (!status) return RGD_E_DEVICE;
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(status, (unsigned long long)limit_ns, nullptr);
    count_launch();
    return check_launch();
}

// Read and clear the sticky device status word of the tensor-memory kernels
// (synchronises the device).
int tmem_status_fetch() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tmem_status, sizeof(int)) != cudaSuccess) {
        (void)cudaGetLastError();
        return -1;
    }
    if (v != 0) {
        const int zero = 0;
        (void)cudaMemcpyToSymbol(g_tmem_status, &zero, sizeof(int));
    }
    return v;
}

}  // namespace attn
}  // namespace rgd
