// extern "C" attention entry points: argument validation, path selection
// (tensor-memory kernels for aligned head_dim 64 / 128, general mma.sync
// kernels otherwise) and workspace layout.
#include "attn_mma.cuh"

namespace rgd {
namespace attn {
int general_fwd(const AttnParams &p, int dtype, cudaStream_t st);
int general_bwd(const AttnParams &p, int dtype, cudaStream_t st);
bool tmem_fwd_eligible(const AttnParams &p);
int tmem_fwd(const AttnParams &p, int dtype, rgd_cache *cache, cudaStream_t st);
int tmem_status_fetch();
bool tmem_bwd_eligible(const AttnParams &p);
int tmem_bwd(const AttnParams &p, int dtype, rgd_cache *cache, float *dq_acc, cudaStream_t st);
int64_t single_pass_acc_offset(int64_t B, int64_t H, int64_t Tq);
int64_t single_pass_acc_bytes(int64_t B, int64_t H, int64_t Tq, int64_t d);
int bounded_wait_selftest(int64_t limit_ns, cudaStream_t st);
int64_t tmem_bwd_workspace_bytes(int64_t B, int64_t H, int64_t Tq);
int build_bias_tiles(const void *bias, int64_t sb, int64_t sh, int64_t sq, int64_t Bb, int64_t Hb, int64_t Tq, int64_t Tk,
                     int dtype, float thr, void *tiles, cudaStream_t st);
}  // namespace attn
}  // namespace rgd

using namespace rgd;
using rgd::attn::AttnParams;

namespace {

bool heads_vec16(const rgd_heads *v) {
    return v && is_aligned(v->ptr, 16) && v->stride_b % 8 == 0 && v->stride_h % 8 == 0 && v->stride_n % 8 == 0;
}

int64_t lse_rows(int64_t Tq) { return (Tq + 63) / 64 * 64; }

int check_common(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_bias *bias, int64_t B,
                 int64_t H, int64_t Tq, int64_t Tk, int64_t d, int dtype) {
    if (!q || !k || !v) return RGD_E_NULL;
    if (dtype != RGD_F16 && dtype != RGD_BF16) return RGD_E_DTYPE;
    if (B < 0 || H < 0 || Tq < 0 || Tk < 0 || d < 0) return RGD_E_INVALID;
    if (d > 128) return RGD_E_SIZE;
    if (B * H > 65535 * 32768LL || Tq > (1LL << 30) || Tk > (1LL << 30) || B > INT32_MAX || H > INT32_MAX)
        return RGD_E_SIZE;
    const bool empty = B == 0 || H == 0 || d == 0;
    if (bias && bias->kind != RGD_BIAS_NONE) {
        if (bias->kind != RGD_BIAS_VECTOR && bias->kind != RGD_BIAS_MATRIX) return RGD_E_BIAS_SHAPE;
        if (bias->dtype != dtype && bias->dtype != RGD_F32) return RGD_E_DTYPE;
        if (!bias->ptr && !empty && Tq > 0 && Tk > 0) return RGD_E_NULL;
    }
    if (!empty) {
        if (Tq > 0 && !q->ptr) return RGD_E_NULL;
        if (Tk > 0 && (!k->ptr || !v->ptr)) return RGD_E_NULL;
    }
    return RGD_OK;
}

void fill_common(AttnParams &p, const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_bias *bias,
                 int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d, float scale, int causal) {
    p.q = q->ptr; p.q_sb = q->stride_b; p.q_sh = q->stride_h; p.q_sn = q->stride_n;
    p.k = k->ptr; p.k_sb = k->stride_b; p.k_sh = k->stride_h; p.k_sn = k->stride_n;
    p.v = v->ptr; p.v_sb = v->stride_b; p.v_sh = v->stride_h; p.v_sn = v->stride_n;
    p.bias_kind = RGD_BIAS_NONE;
    if (bias && bias->kind != RGD_BIAS_NONE) {
        p.bias = bias->ptr;
        p.b_sb = bias->stride_b;
        p.b_sh = bias->stride_h;
        p.b_sq = bias->kind == RGD_BIAS_MATRIX ? bias->stride_q : 0;
        p.bias_kind = bias->kind;
        p.bias_f32 = bias->dtype == RGD_F32;
        if (bias->kind == RGD_BIAS_MATRIX && !causal && bias->dtype != RGD_F32 && is_aligned(bias->tiles, 16))
            p.tiles = reinterpret_cast<const uint16_t *>(bias->tiles);
    }
    p.B = (int)B; p.H = (int)H; p.Tq = (int)Tq; p.Tk = (int)Tk; p.d = (int)d;
    p.Tq_rounded = (int)lse_rows(Tq);
    p.causal = causal ? 1 : 0;
    p.scale = scale;
    const bool dvec = d % 8 == 0;
    p.vec_q = dvec && heads_vec16(q);
    p.vec_k = dvec && heads_vec16(k);
    p.vec_v = dvec && heads_vec16(v);
}

void fill_fwd(AttnParams &p, const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_bias *bias,
              const rgd_heads *o, int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d, float scale, int causal) {
    fill_common(p, q, k, v, bias, B, H, Tq, Tk, d, scale, causal);
    p.out_o = o->ptr; p.o_sb = o->stride_b; p.o_sh = o->stride_h; p.o_sn = o->stride_n;
    p.vec_o = d % 8 == 0 && heads_vec16(o);
}

void fill_bwd(AttnParams &p, const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_bias *bias,
              const rgd_heads *o, const rgd_heads *d_o, const rgd_heads *dq, const rgd_heads *dk, const rgd_heads *dv,
              int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d, float scale, int causal) {
    fill_common(p, q, k, v, bias, B, H, Tq, Tk, d, scale, causal);
    p.o = o->ptr; p.o_sb = o->stride_b; p.o_sh = o->stride_h; p.o_sn = o->stride_n;
    p.d_o = d_o->ptr; p.do_sb = d_o->stride_b; p.do_sh = d_o->stride_h; p.do_sn = d_o->stride_n;
    p.dq = dq->ptr; p.dq_sb = dq->stride_b; p.dq_sh = dq->stride_h; p.dq_sn = dq->stride_n;
    p.dk = dk->ptr; p.dk_sb = dk->stride_b; p.dk_sh = dk->stride_h; p.dk_sn = dk->stride_n;
    p.dv = dv->ptr; p.dv_sb = dv->stride_b; p.dv_sh = dv->stride_h; p.dv_sn = dv->stride_n;
    const bool dvec = d % 8 == 0;
    p.vec_o = dvec && heads_vec16(o);
    p.vec_do = dvec && heads_vec16(d_o);
    p.vec_dq = dvec && heads_vec16(dq);
    p.vec_dk = dvec && heads_vec16(dk);
    p.vec_dv = dvec && heads_vec16(dv);
}

}  // namespace

extern "C" int64_t rgd_attn_lse_rows(int64_t Tq) { return Tq < 0 ? RGD_E_INVALID : lse_rows(Tq); }

extern "C" int rgd_device_status(void) {
    const int v = attn::tmem_status_fetch();
    if (v < 0) return RGD_E_CUDA_BASE;
    return v == 0 ? RGD_OK : RGD_E_TIMEOUT;
}

extern "C" int rgd_attn_fwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_bias *bias,
                            const rgd_heads *o, float *lse, int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d,
                            float softmax_scale, int causal, int dtype, rgd_cache *cache, void *stream) {
    if (int e = check_common(q, k, v, bias, B, H, Tq, Tk, d, dtype)) return e;
    if (!o) return RGD_E_NULL;
    const bool work = B > 0 && H > 0 && Tq > 0;
    if (work && (!lse || (d > 0 && !o->ptr))) return RGD_E_NULL;
    AttnParams p{};
    fill_fwd(p, q, k, v, bias, o, B, H, Tq, Tk, d, softmax_scale, causal);
    p.lse = lse;
    if (work && attn::tmem_fwd_eligible(p)) {
        const int rc = attn::tmem_fwd(p, dtype, cache, (cudaStream_t)stream);
        if (rc != attn::TMEM_NOT_TAKEN) return rc;
    }
    return attn::general_fwd(p, dtype, (cudaStream_t)stream);
}

extern "C" int rgd_attn_fwd_uses_tmem(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_heads *o,
                                      int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d, float softmax_scale,
                                      int dtype) {
    if (check_common(q, k, v, nullptr, B, H, Tq, Tk, d, dtype) != RGD_OK || !o) return 0;
    AttnParams p{};
    fill_fwd(p, q, k, v, nullptr, o, B, H, Tq, Tk, d, softmax_scale, 0);
    return (B > 0 && H > 0 && Tq > 0 && attn::tmem_fwd_eligible(p)) ? 1 : 0;
}

extern "C" int64_t rgd_attn_bwd_workspace_bytes(int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d, int dtype) {
    (void)Tk; (void)d; (void)dtype;
    if (B < 0 || H < 0 || Tq < 0) return RGD_E_INVALID;
    // general path: delta [B,H,Tq_rounded]; tensor-memory path: lse*log2e and delta*scale, [B,H,Tq128] each
    const int64_t general = B * H * lse_rows(Tq) * (int64_t)sizeof(float);
    const int64_t tmem = attn::tmem_bwd_workspace_bytes(B, H, Tq);
    return general > tmem ? general : tmem;
}

extern "C" int64_t rgd_attn_bwd_single_pass_workspace_bytes(int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d,
                                                            int dtype) {
    const int64_t base = rgd_attn_bwd_workspace_bytes(B, H, Tq, Tk, d, dtype);
    if (base < 0) return base;
    const int64_t acc = attn::single_pass_acc_bytes(B, H, Tq, d);
    if (acc == 0) return 0;
    return attn::single_pass_acc_offset(B, H, Tq) + acc;
}

extern "C" int rgd_attn_bwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_bias *bias,
                            const rgd_heads *o, const float *lse, const rgd_heads *d_o, const rgd_heads *dq,
                            const rgd_heads *dk, const rgd_heads *dv, int64_t B, int64_t H, int64_t Tq, int64_t Tk,
                            int64_t d, float softmax_scale, int causal, int dtype, void *workspace,
                            int64_t workspace_bytes, rgd_cache *cache, void *stream) {
    return rgd_attn_bwd_dbias(q, k, v, bias, o, lse, d_o, dq, dk, dv, nullptr, B, H, Tq, Tk, d, softmax_scale, causal, dtype,
                              workspace, workspace_bytes, cache, stream);
}

extern "C" int rgd_attn_bwd_dbias(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_bias *bias,
                                  const rgd_heads *o, const float *lse, const rgd_heads *d_o, const rgd_heads *dq,
                                  const rgd_heads *dk, const rgd_heads *dv, const rgd_bias *dbias, int64_t B, int64_t H,
                                  int64_t Tq, int64_t Tk, int64_t d, float softmax_scale, int causal, int dtype,
                                  void *workspace, int64_t workspace_bytes, rgd_cache *cache, void *stream) {
    if (int e = check_common(q, k, v, bias, B, H, Tq, Tk, d, dtype)) return e;
    const bool want_dbias = dbias && dbias->kind != RGD_BIAS_NONE;
    if (want_dbias) {
        // same kind as the bias; vector: dense fp32 [B, H, Tk]; matrix: the tensor dtype, unit key stride
        if (!bias || bias->kind != dbias->kind) return RGD_E_BIAS_SHAPE;
        if (dbias->kind == RGD_BIAS_VECTOR) {
            if (dbias->dtype != RGD_F32) return RGD_E_DTYPE;
            if (dbias->stride_h != Tk || dbias->stride_b != H * Tk) return RGD_E_STRIDE;
        } else {
            if (dbias->dtype != dtype) return RGD_E_DTYPE;
            if (dbias->stride_q < Tk || dbias->stride_h < 0 || dbias->stride_b < 0) return RGD_E_STRIDE;
        }
        if (!dbias->ptr && B > 0 && H > 0 && Tq > 0 && Tk > 0) return RGD_E_NULL;
    }
    if (!o || !d_o || !dq || !dk || !dv) return RGD_E_NULL;
    const bool work = B > 0 && H > 0 && d > 0;
    if (work && Tq > 0 && (!o->ptr || !d_o->ptr || !dq->ptr || !lse)) return RGD_E_NULL;
    if (work && Tk > 0 && (!dk->ptr || !dv->ptr)) return RGD_E_NULL;
    const int64_t need = rgd_attn_bwd_workspace_bytes(B, H, Tq, Tk, d, dtype);
    if (need > 0 && (!workspace || workspace_bytes < need)) return RGD_E_WORKSPACE;
    if (need > 0 && !is_aligned(workspace, 16)) return RGD_E_STRIDE;
    AttnParams p{};
    fill_bwd(p, q, k, v, bias, o, d_o, dq, dk, dv, B, H, Tq, Tk, d, softmax_scale, causal);
    p.lse = const_cast<float *>(lse);
    p.delta = reinterpret_cast<float *>(workspace);
    if (want_dbias && B > 0 && H > 0 && Tk > 0) {
        if (dbias->kind == RGD_BIAS_VECTOR &&
            cudaMemsetAsync(const_cast<void *>(dbias->ptr), 0, (size_t)(B * H * Tk) * sizeof(float), (cudaStream_t)stream) != cudaSuccess)
            return RGD_E_DEVICE;
        p.tiles = nullptr;      // a skipped tile's gradient entries would not be written
        if (work && Tq > 0) {
            p.dbias = const_cast<void *>(dbias->ptr);
            p.db_sb = dbias->stride_b; p.db_sh = dbias->stride_h;
            p.db_sq = dbias->kind == RGD_BIAS_MATRIX ? dbias->stride_q : 0;
            p.dbias_vec = is_aligned(dbias->ptr, 16) && p.db_sb % 8 == 0 && p.db_sh % 8 == 0 && p.db_sq % 8 == 0;
        }
    }
    if (work && attn::tmem_bwd_eligible(p)) {
        // a workspace with room for the fp32 dQ accumulator selects the single-pass form
        float *dq_acc = nullptr;
        const int64_t single = rgd_attn_bwd_single_pass_workspace_bytes(B, H, Tq, Tk, d, dtype);
        if (single > 0 && workspace_bytes >= single && is_aligned(workspace, 256))
            dq_acc = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + attn::single_pass_acc_offset(B, H, Tq));
        const int rc = attn::tmem_bwd(p, dtype, cache, dq_acc, (cudaStream_t)stream);
        if (rc != attn::TMEM_NOT_TAKEN) return rc;
    }
    return attn::general_bwd(p, dtype, (cudaStream_t)stream);
}

extern "C" int rgd_attn_bwd_uses_tmem(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v, const rgd_heads *o,
                                      const rgd_heads *d_o, const rgd_heads *dq, const rgd_heads *dk,
                                      const rgd_heads *dv, int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d,
                                      int dtype) {
    if (check_common(q, k, v, nullptr, B, H, Tq, Tk, d, dtype) != RGD_OK || !o || !d_o || !dq || !dk || !dv) return 0;
    AttnParams p{};
    fill_bwd(p, q, k, v, nullptr, o, d_o, dq, dk, dv, B, H, Tq, Tk, d, 1.f, 0);
    return (B > 0 && H > 0 && d > 0 && attn::tmem_bwd_eligible(p)) ? 1 : 0;
}

extern "C" int64_t rgd_attn_bias_tiles_bytes(int64_t B, int64_t H, int64_t Tq, int64_t Tk) {
    if (B < 0 || H < 0 || Tq < 0 || Tk < 0) return RGD_E_INVALID;
    return attn::tile_layout(B, H, Tq, Tk).total_bytes;
}

extern "C" int rgd_attn_bias_tiles_build(const rgd_bias *bias, int64_t B, int64_t H, int64_t Tq, int64_t Tk,
                                         float threshold, void *tiles, int64_t tiles_bytes, void *stream) {
    if (!bias || !tiles) return RGD_E_NULL;
    if (B < 0 || H < 0 || Tq < 0 || Tk < 0 || !(threshold < 0.f)) return RGD_E_INVALID;
    if (bias->kind != RGD_BIAS_MATRIX) return RGD_E_BIAS_SHAPE;
    if (bias->dtype != RGD_F16 && bias->dtype != RGD_BF16) return RGD_E_DTYPE;
    if (bias->stride_b < 0 || bias->stride_h < 0 || bias->stride_q < Tk) return RGD_E_STRIDE;
    if (!is_aligned(tiles, 16)) return RGD_E_STRIDE;
    if (tiles_bytes < rgd_attn_bias_tiles_bytes(B, H, Tq, Tk)) return RGD_E_WORKSPACE;
    if (B == 0 || H == 0 || Tq == 0 || Tk == 0) return RGD_OK;
    if (!bias->ptr) return RGD_E_NULL;
    const int64_t Bb = bias->stride_b == 0 ? 1 : B, Hb = bias->stride_h == 0 ? 1 : H;
    return attn::build_bias_tiles(bias->ptr, bias->stride_b, bias->stride_h, bias->stride_q, Bb, Hb, Tq, Tk, bias->dtype,
                                  threshold, tiles, (cudaStream_t)stream);
}

extern "C" int rgd_selftest_bounded_wait(int64_t limit_ns, void *stream) {
    if (limit_ns < 1000 || limit_ns > 100000000) return RGD_E_INVALID;      // 1 us .. 100 ms
    return attn::bounded_wait_selftest(limit_ns, (cudaStream_t)stream);
}
