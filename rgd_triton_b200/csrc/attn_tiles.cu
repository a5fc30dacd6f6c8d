// Tile lists of a matrix attention bias: one pass over the bias finds the 128 x 128 tiles whose
// every element is <= a threshold (the -1e4 "masked" convention of additive masks): with the
// softmax of a row dominated by some unmasked key, such a tile contributes exp(-1e4 + ...) = 0
// exactly in fp32, so the kernels that stage the bias by TMA may skip it: no K / V / bias tile
// load, no MMAs, no exponentials.  A query block is only trimmed when EVERY one of its rows has
// at least one element >= threshold / 2 (a row with nothing but masked keys is a softmax over
// the raw scores, where a skipped tile would change the result): otherwise its list is full.
// The reference has only the dense form (flash_attn_triton_cached.py:151-175, 781-788).
#include "attn_mma.cuh"

namespace rgd {
namespace attn {

// One CTA per (128-query block, bias head, bias batch); 256 threads: thread = (row, half of the
// tile's 128 columns).  Writes one byte per key block: 1 = visit.
template <typename T>
__global__ void __launch_bounds__(256) bias_tile_scan_kernel(const T *__restrict__ bias, int64_t sb, int64_t sh, int64_t sq,
                                                             int Tq, int Tk, int nqb, int nkb, float thr, int vec_ok,
                                                             uint8_t *__restrict__ active) {
    const int qb = blockIdx.x;
    const int64_t slice = (int64_t)blockIdx.z * gridDim.y + blockIdx.y;
    const T *base = bias + (int64_t)blockIdx.z * sb + (int64_t)blockIdx.y * sh;
    uint8_t *out = active + (slice * nqb + qb) * nkb;
    const int row = qb * 128 + ((int)threadIdx.x >> 1), half = (int)threadIdx.x & 1;
    const float alive_thr = 0.5f * thr;
    bool row_alive = false;
    for (int kb = 0; kb < nkb; ++kb) {
        bool live = false;
        const int c0 = kb * 128 + half * 64;
        if (row < Tq && c0 < Tk) {
            const T *src = base + (int64_t)row * sq + c0;
            if (vec_ok && c0 + 64 <= Tk) {
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const Vec<T, 8> v8 = load_vec_stream<T, 8>(src + 8 * c);
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const float v = to_f32<T>(v8.v[e]);
                        live |= v > thr;
                        row_alive |= v >= alive_thr;
                    }
                }
            } else {
                for (int i = 0; i < 64 && c0 + i < Tk; ++i) {
                    const float v = to_f32<T>(src[i]);
                    live |= v > thr;
                    row_alive |= v >= alive_thr;
                }
            }
        }
        const int any = __syncthreads_or(live ? 1 : 0);
        if (threadIdx.x == 0) out[kb] = any ? 1 : 0;
    }
    // a row's two threads each saw half of its columns
    row_alive |= __shfl_xor_sync(0xffffffffu, row_alive ? 1 : 0, 1) != 0;
    const int dead_row = __syncthreads_or((row < Tq && !row_alive) ? 1 : 0);
    if (dead_row)
        for (int kb = threadIdx.x; kb < nkb; kb += 256) out[kb] = 1;
}

// One CTA per bias slice: the three list sets from the bitmap.
__global__ void __launch_bounds__(128) bias_tile_lists_kernel(const uint8_t *__restrict__ active, uint16_t *__restrict__ w,
                                                              TileLayout L) {
    const int64_t s = blockIdx.x;
    const uint8_t *a = active + s * L.nqb * L.nkb;
    for (int qb = threadIdx.x; qb < L.nqb; qb += blockDim.x) {
        uint16_t *lst = w + L.qlist + (s * L.nqb + qb) * L.nkb;
        int n = 0;
        for (int kb = 0; kb < L.nkb; ++kb)
            if (a[qb * L.nkb + kb]) lst[n++] = (uint16_t)kb;
        w[L.qcnt + s * L.nqb + qb] = (uint16_t)n;
    }
    for (int q2 = threadIdx.x; q2 < L.nq2; q2 += blockDim.x) {
        uint16_t *lst = w + L.q2list + (s * L.nq2 + q2) * L.nkb;
        const int qa = 2 * q2, qb = 2 * q2 + 1 < L.nqb ? 2 * q2 + 1 : 2 * q2;
        int n = 0;
        for (int kb = 0; kb < L.nkb; ++kb)
            if (a[qa * L.nkb + kb] | a[qb * L.nkb + kb]) lst[n++] = (uint16_t)kb;
        w[L.q2cnt + s * L.nq2 + q2] = (uint16_t)n;
    }
    for (int kb = threadIdx.x; kb < L.nkb; kb += blockDim.x) {
        uint16_t *lst = w + L.klist + (s * L.nkb + kb) * L.nqb;
        int n = 0;
        for (int qb = 0; qb < L.nqb; ++qb)
            if (a[qb * L.nkb + kb]) lst[n++] = (uint16_t)qb;
        w[L.kcnt + s * L.nkb + kb] = (uint16_t)n;
    }
}

// bias: matrix kind in a 16-bit dtype.  Bb / Hb: 1 where the bias is broadcast (stride 0).
int build_bias_tiles(const void *bias, int64_t sb, int64_t sh, int64_t sq, int64_t Bb, int64_t Hb, int64_t Tq, int64_t Tk,
                     int dtype, float thr, void *tiles, cudaStream_t st) {
    const TileLayout L = tile_layout(Bb, Hb, Tq, Tk);
    if (L.slices == 0 || L.nqb == 0 || L.nkb == 0) return RGD_OK;
    if (L.nkb > 65535 || L.nqb > 65535 || Hb > 65535 || Bb > 65535) return RGD_E_SIZE;
    uint16_t *words = reinterpret_cast<uint16_t *>(tiles);
    uint8_t *bitmap = reinterpret_cast<uint8_t *>(tiles) + L.words * 2;
    const int vec_ok = is_aligned(bias, 16) && sb % 8 == 0 && sh % 8 == 0 && sq % 8 == 0;
    dim3 grid(L.nqb, (unsigned)Hb, (unsigned)Bb);
    if (dtype == RGD_BF16)
        bias_tile_scan_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16 *>(bias), sb, sh, sq,
                                                                    (int)Tq, (int)Tk, L.nqb, L.nkb, thr, vec_ok, bitmap);
    else
        bias_tile_scan_kernel<__half><<<grid, 256, 0, st>>>(reinterpret_cast<const __half *>(bias), sb, sh, sq, (int)Tq,
                                                             (int)Tk, L.nqb, L.nkb, thr, vec_ok, bitmap);
    count_launch();
    if (int e = check_launch()) return e;
    bias_tile_lists_kernel<<<(unsigned)L.slices, 128, 0, st>>>(bitmap, words, L);
    count_launch();
    return check_launch();
}

}  // namespace attn
}  // namespace rgd
