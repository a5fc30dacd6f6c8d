/*
 * rgd_b200.h — C ABI of librgd_b200.so: hand-written sm_100a CUDA kernels for the
 * rgd_triton operator set (row L2 / RMS norms, per-head LayerNorm, rotary
 * embedding, fused LayerNorm+rotary, FlashAttention with additive bias).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer on the current device.  The caller owns
 *     every buffer; the library allocates no device memory.
 *   - Strides are in ELEMENTS.  The innermost (channel / head_dim) stride is 1.
 *   - Sizes are int64_t; dtype codes are RGD_F32 / RGD_F16 / RGD_BF16.
 *   - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *   - Return value: 0 success; <0 argument error (see RGD_E_*); >=1000 is
 *     1000 + cudaError_t; RGD_E_TIMEOUT a bounded device-side wait that ran out.
 *     Argument errors correspond to the AssertionError / RuntimeError the
 *     reference's host wrappers raise; the Python layer re-raises them as such.
 *   - All entry points are re-entrant.  Process-wide state: a memo of the
 *     per-kernel cudaFuncSetAttribute opt-ins for large shared memory and of
 *     occupancy queries (each made once per device and kernel), the launch
 *     counter, the sticky status word of the bounded device-side waits, and the
 *     fixed scratch of rgd_rmsnorm_bwd_static.
 *
 * Each declaration cites the reference interface (file:line inside the
 * rgd_triton project) whose launch it replaces.
 */
#ifndef RGD_B200_H
#define RGD_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- dtype codes ------------------------------------------------------- */
#define RGD_F32  0
#define RGD_F16  1
#define RGD_BF16 2

/* ---- status codes ------------------------------------------------------ */
#define RGD_OK              0
#define RGD_E_INVALID      -1   /* generic bad argument (shape mismatch, negative size) */
#define RGD_E_DTYPE        -2   /* dtype not supported by this operator                 */
#define RGD_E_SIZE         -3   /* size outside the operator's limits (e.g. head_dim)   */
#define RGD_E_STRIDE       -4   /* stride / alignment the kernel cannot address         */
#define RGD_E_NULL         -5   /* required pointer is NULL                             */
#define RGD_E_WORKSPACE    -6   /* caller workspace too small                           */
#define RGD_E_DEVICE       -7   /* current device is not compute capability 10.x        */
#define RGD_E_BIAS_SHAPE   -8   /* bias is neither (1,Tk) "vector" nor (Tq,Tk) "matrix" */
#define RGD_E_TIMEOUT    2001   /* bounded device-side wait expired                     */
#define RGD_E_CUDA_BASE  1000   /* 1000 + cudaError_t                                   */

/* ---- tensor views ------------------------------------------------------ */
/* [B, N, C] row tensor, channel stride 1. */
typedef struct rgd_rows {
    void   *ptr;
    int64_t stride_b;
    int64_t stride_n;
} rgd_rows;

/* 4-D head tensor addressed as (batch, head, token, channel) whatever its
 * memory order: a [B,N,H,d] tensor passes stride_h = stride(2), stride_n =
 * stride(1); a [B,H,N,d] tensor passes them the other way round.  This is the
 * (B,H,N) stride triple of head_layernorm_cached.py:216-231. */
typedef struct rgd_heads {
    void   *ptr;
    int64_t stride_b;
    int64_t stride_h;
    int64_t stride_n;
} rgd_heads;

/* ---- library ----------------------------------------------------------- */
/* 1 if `device` is compute capability 10.x, 0 if not, <0 on error. */
int         rgd_device_supported(int device);
/* Static string for a status code returned by any entry point. */
const char *rgd_status_string(int status);
/* ABI version of this header (bumped on any signature change). */
int         rgd_abi_version(void);
/* Number of kernels this library has launched in the calling process. */
int64_t     rgd_launch_count(void);
/* Sticky status of the tensor-memory kernels' bounded device-side waits:
 * RGD_OK, or RGD_E_TIMEOUT if a wait ran out since the last call (the flag is
 * cleared by the call).  Synchronises the device; meant for tests, smoke
 * checks and debugging, not for the per-step path. */
int         rgd_device_status(void);

/* Test hook for the bounded device-side waits (no counterpart in the
 * reference): launches one thread that waits, for at most `limit_ns`
 * (1 us .. 100 ms), on a barrier nothing ever arrives at.  The wait gives up,
 * records itself in the status word and the kernel returns normally, so the
 * next rgd_device_status() reports RGD_E_TIMEOUT once and RGD_OK afterwards.
 * Nothing traps, faults or spins without a limit. */
int         rgd_selftest_bounded_wait(int64_t limit_ns, void *stream);

/* ---- launch-plan cache -------------------------------------------------- */
/* What `enable_cache` means here.  The reference keeps the compiled Triton
 * kernel handle of the first launch in the module's cache slot and relaunches
 * it directly (rgd_triton/ops.py:12-24, e.g.
 * flash_attn_triton_cached.py:805-836,878-879).  This library has nothing to
 * compile at run time; what costs host time per attention call is encoding the
 * TMA tensor-map descriptors.  An rgd_cache holds the descriptors of the calls
 * it has seen, keyed on base pointer + extents + strides + box + dtype, so a
 * repeated call copies them instead of re-encoding, and a call whose tensors
 * moved or changed shape misses and re-encodes (it can never launch with a
 * stale descriptor, unlike the reference's frozen constexprs).  The handle is
 * host memory only; pass NULL wherever a cache is accepted to run without. */
typedef struct rgd_cache rgd_cache;
rgd_cache  *rgd_cache_create(void);                 /* NULL if out of host memory */
void        rgd_cache_destroy(rgd_cache *cache);    /* NULL is allowed            */
/* Counters of the cache (any of the three pointers may be NULL). */
int         rgd_cache_stats(rgd_cache *cache, int64_t *hits, int64_t *misses,
                            int64_t *entries);

/* ---- row L2 normalise: y = x / max(||x||, eps) ------------------------- */
/* Replaces _norm_fwd / _fused_norm_fwd (l2normalize_cached.py:237-318,
 * fused_l2normalize_cached.py:251-345).  nstreams is 1 or 2; with 2 both
 * tensors are processed by ONE launch (the reference's virtual-tensor fusion).
 * x[s], y[s]: views of [B, N[s], C[s]]. */
int rgd_l2norm_fwd(int nstreams, const rgd_rows *x, const rgd_rows *y,
                   const int64_t *N, const int64_t *C, int64_t B,
                   float eps, int dtype, void *stream);
/* Replaces _norm_bwd / _fused_norm_bwd (l2normalize_cached.py:321-399,
 * fused_l2normalize_cached.py:348-461).  The row scale is recomputed from x,
 * so no statistics buffer is passed. */
int rgd_l2norm_bwd(int nstreams, const rgd_rows *x, const rgd_rows *dy,
                   const rgd_rows *dx, const int64_t *N, const int64_t *C,
                   int64_t B, float eps, int dtype, void *stream);

/* ---- row RMS norm with affine weight: y = x * rsqrt(mean(x^2)+eps) * w -- */
/* Replaces _rms_fwd / _fused_rms_fwd (rmsnorm_cached.py:319-403,
 * fused_rmsnorm_cached.py:385-487).  w[s] points at [B or 1, C[s]] weights;
 * w_stride_b[s] is 0 for a weight shared by all batches. */
int rgd_rmsnorm_fwd(int nstreams, const rgd_rows *x, const void *const *w,
                    const int64_t *w_stride_b, const rgd_rows *y,
                    const int64_t *N, const int64_t *C, int64_t B,
                    float eps, int x_dtype, int w_dtype, void *stream);
/* Bytes of scratch rgd_rmsnorm_bwd needs (per-CTA fp32 dweight partials). */
int64_t rgd_rmsnorm_bwd_workspace_bytes(int nstreams, const int64_t *N,
                                        const int64_t *C, int64_t B);
/* Replaces _rms_bwd / _fused_rms_bwd plus the dweight reduce kernel
 * (rmsnorm_cached.py:406-569, fused_rmsnorm_cached.py:490-722).  dw[s] is
 * [B, C[s]] when dw_per_batch[s] != 0, else [C[s]] — the sum over batches
 * is taken in fp32 and rounded once to w_dtype.  dweight is deterministic:
 * per-CTA partials in `workspace`, then a fixed-order reduce. */
int rgd_rmsnorm_bwd(int nstreams, const rgd_rows *x, const void *const *w,
                    const int64_t *w_stride_b, const rgd_rows *dy,
                    const rgd_rows *dx, void *const *dw,
                    const int *dw_per_batch, const int64_t *N,
                    const int64_t *C, int64_t B, float eps, int x_dtype,
                    int w_dtype, void *workspace, int64_t workspace_bytes,
                    void *stream);

/* Capacity of the built-in scratch of rgd_rmsnorm_bwd_static: 16 MiB of device
 * memory per GPU, held from library load to process exit. */
#define RGD_RMSNORM_BWD_STATIC_SCRATCH_BYTES (16ll << 20)
/* rgd_rmsnorm_bwd for callers that cannot allocate device memory (no
 * counterpart in the reference, which allocates its scratch with torch on
 * every call).  Same arguments and results as rgd_rmsnorm_bwd minus the
 * workspace: the dweight partial rows go to a fixed device array inside the
 * library.  The call itself allocates nothing — no cudaMalloc / cudaFree, no
 * allocating library routine.
 *   - Limit: rgd_rmsnorm_bwd_workspace_bytes(...) for the call must not exceed
 *     RGD_RMSNORM_BWD_STATIC_SCRATCH_BYTES, otherwise RGD_E_WORKSPACE is
 *     returned and nothing is launched (e.g. two streams of 3072 channels fit,
 *     two streams of 4096 channels do not).
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress, with that device current); make that first call
 *     before starting any stream capture on the device.
 *   - All calls on a device share the one array, which keeps the previous
 *     call's contents; nothing in it needs clearing between calls, but two
 *     calls that overlap on the GPU (different streams) race on it. */
int rgd_rmsnorm_bwd_static(int nstreams, const rgd_rows *x, const void *const *w,
                           const int64_t *w_stride_b, const rgd_rows *dy,
                           const rgd_rows *dx, void *const *dw,
                           const int *dw_per_batch, const int64_t *N,
                           const int64_t *C, int64_t B, float eps, int x_dtype,
                           int w_dtype, void *stream);

/* ---- per-head LayerNorm (no affine) on Q and K in one launch ----------- */
/* Replaces _fused_ln_qk_fwd / _fused_ln_qk_bwd
 * (head_layernorm_cached.py:204-308, :310-408).  head_dim <= 256. */
int rgd_headln_fwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *qo,
                   const rgd_heads *ko, int64_t B, int64_t H, int64_t Nq,
                   int64_t Nk, int64_t head_dim, float eps, int dtype,
                   void *stream);
int rgd_headln_bwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *dqo,
                   const rgd_heads *dko, const rgd_heads *dq,
                   const rgd_heads *dk, int64_t B, int64_t H, int64_t Nq,
                   int64_t Nk, int64_t head_dim, float eps, int dtype,
                   void *stream);

/* ---- rotary embedding on Q and K in one launch ------------------------- */
/* Replaces combined_rope_fn (head_rope_cached.py:160-275).  pos is
 * [2, P, R] (index 0 = sin, 1 = cos) with element strides pos_stride_s /
 * pos_stride_n; the first R channels of the first cut_q / cut_k tokens are
 * rotated as interleaved pairs, everything else is copied.  transposed != 0
 * applies the inverse rotation (the backward pass).  Arithmetic is done in
 * the promoted type of x and pos, as the reference does: pos_dtype must be
 * either x_dtype or RGD_F32.  qo may alias q (in place).  head_dim <= 128. */
int rgd_rope(const rgd_heads *q, const rgd_heads *k, const void *pos,
             int64_t pos_stride_s, int64_t pos_stride_n, const rgd_heads *qo,
             const rgd_heads *ko, int64_t B, int64_t H, int64_t Nq, int64_t Nk,
             int64_t head_dim, int64_t P, int64_t R, int64_t cut_q,
             int64_t cut_k, int transposed, int x_dtype, int pos_dtype,
             void *stream);

/* ---- fused per-head LayerNorm -> rotary -------------------------------- */
/* Replaces _fused_rope_ln_qk_fwd / _fused_rope_ln_qk_bwd
 * (fused_ln_rope_cached.py:382-516, :518-647).  fp32 arithmetic throughout,
 * one rounding on store. */
int rgd_lnrope_fwd(const rgd_heads *q, const rgd_heads *k, const void *pos,
                   int64_t pos_stride_s, int64_t pos_stride_n,
                   const rgd_heads *qo, const rgd_heads *ko, int64_t B,
                   int64_t H, int64_t Nq, int64_t Nk, int64_t head_dim,
                   int64_t P, int64_t R, int64_t cut_q, int64_t cut_k,
                   float eps, int x_dtype, int pos_dtype, void *stream);
int rgd_lnrope_bwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *dqo,
                   const rgd_heads *dko, const void *pos, int64_t pos_stride_s,
                   int64_t pos_stride_n, const rgd_heads *dq,
                   const rgd_heads *dk, int64_t B, int64_t H, int64_t Nq,
                   int64_t Nk, int64_t head_dim, int64_t P, int64_t R,
                   int64_t cut_q, int64_t cut_k, float eps, int x_dtype,
                   int pos_dtype, void *stream);

/* ---- FlashAttention ---------------------------------------------------- */
#define RGD_BIAS_NONE   0
#define RGD_BIAS_VECTOR 1   /* last two dims (1, Tk)  */
#define RGD_BIAS_MATRIX 2   /* last two dims (Tq, Tk) */

/* Additive bias, logically (B, H, Tq, Tk) with stride 0 on broadcast dims,
 * innermost stride 1 (flash_attn_triton_cached.py:771-788). */
typedef struct rgd_bias {
    const void *ptr;
    int64_t stride_b;
    int64_t stride_h;
    int64_t stride_q;   /* ignored for RGD_BIAS_VECTOR */
    int     kind;       /* RGD_BIAS_*                   */
    int     dtype;      /* the q dtype or RGD_F32       */
    const void *tiles;  /* null, or the tile lists rgd_attn_bias_tiles_build
                           made for exactly this tensor (RGD_BIAS_MATRIX only) */
} rgd_bias;

/* Block-sparse skip of masked bias tiles (the reference has only the dense
 * form, flash_attn_triton_cached.py:151-175).  rgd_attn_bias_tiles_build reads
 * a matrix bias once (16-bit dtype, dims as for the attention call, stride 0 on
 * broadcast dims) and records which 128 x 128 tiles have an element above
 * `threshold` (the additive-mask convention is -1e4; use -9984, which is what
 * bf16 stores for it, so that masks of either 16-bit type count).  Passed back through
 * rgd_bias.tiles, the tensor-memory kernels skip the other tiles: their
 * probabilities are exp(-1e4 + ...) = 0 exactly in fp32, so the results are
 * bit-identical PROVIDED |score * scale| stays far below |threshold| / 2.  A
 * query block with a row that has no element >= threshold / 2 keeps its full
 * list.  The lists are ignored with a causal mask, by the general kernels and by
 * rgd_attn_bwd_dbias.  They describe the VALUES of the bias: rebuild after the
 * tensor changes.  `tiles` must hold rgd_attn_bias_tiles_bytes(B, H, Tq, Tk)
 * bytes, 16-byte aligned. */
int64_t rgd_attn_bias_tiles_bytes(int64_t B, int64_t H, int64_t Tq, int64_t Tk);
int rgd_attn_bias_tiles_build(const rgd_bias *bias, int64_t B, int64_t H,
                              int64_t Tq, int64_t Tk, float threshold,
                              void *tiles, int64_t tiles_bytes, void *stream);

/* Rows of the log-sum-exp buffer: Tq rounded up to a multiple of 64, the
 * same rule as flash_attn_triton_cached.py:790-792. */
int64_t rgd_attn_lse_rows(int64_t Tq);

/* O = softmax(Q K^T * scale + bias) V and LSE.  Replaces
 * _flash_attn_forward (flash_attn_triton_cached.py:758-882).
 * q: (B,H,Tq,d) view; k, v: (B,H,Tk,d) views; o: like q; lse: fp32
 * [B, H, rgd_attn_lse_rows(Tq)].  dtype RGD_F16 / RGD_BF16, d <= 128.
 * causal masks key j > query i (top-left aligned, as the reference). */
int rgd_attn_fwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v,
                 const rgd_bias *bias, const rgd_heads *o, float *lse,
                 int64_t B, int64_t H, int64_t Tq, int64_t Tk, int64_t d,
                 float softmax_scale, int causal, int dtype, rgd_cache *cache,
                 void *stream);

/* Scratch bytes for rgd_attn_bwd: one fp32 row of delta = rowsum(O * dO) per
 * (batch, head) on the general path; on the tensor-memory path two fp32 rows
 * per (batch, head), lse * log2(e) and delta * scale, each Tq rounded up to
 * 128.  With exactly this much, no fp32 dQ accumulator is used on either path. */
int64_t rgd_attn_bwd_workspace_bytes(int64_t B, int64_t H, int64_t Tq,
                                     int64_t Tk, int64_t d, int dtype);

/* Scratch bytes that select the single-pass backward (0 where there is none:
 * it exists for head_dim 64 on the tensor-memory path, without tile lists and
 * without a bias gradient): the bytes above, rounded up to 256, plus an fp32 dQ
 * accumulator of B * H * Tq (rounded up to 128) * d elements, which the entry
 * point zeroes itself.  Given at least this much 256-byte aligned workspace,
 * rgd_attn_bwd evaluates S, dP and the exponentials once per tile pair and adds
 * the dQ partial tiles into the accumulator with vector reductions, the scheme
 * of the reference's sequence-parallel backward (tl.atomic_add into dq,
 * flash_attn_triton_cached.py:556-561): dK and dV are bit-reproducible, dQ may
 * differ in its last bits from run to run (the reference's own test allows
 * that, tests/test_flash_attn.py:341-388).  Given less, rgd_attn_bwd runs the
 * two-kernel form, in which dQ is bit-reproducible too. */
int64_t rgd_attn_bwd_single_pass_workspace_bytes(int64_t B, int64_t H,
                                                 int64_t Tq, int64_t Tk,
                                                 int64_t d, int dtype);

/* dQ, dK, dV given dO.  Replaces _flash_attn_backward, including the
 * delta = rowsum(O * dO) pre-pass (flash_attn_triton_cached.py:885-1075).
 * The bias gradient (which the reference refuses, :1107) comes from
 * rgd_attn_bwd_dbias. */
int rgd_attn_bwd(const rgd_heads *q, const rgd_heads *k, const rgd_heads *v,
                 const rgd_bias *bias, const rgd_heads *o, const float *lse,
                 const rgd_heads *d_o, const rgd_heads *dq,
                 const rgd_heads *dk, const rgd_heads *dv, int64_t B,
                 int64_t H, int64_t Tq, int64_t Tk, int64_t d,
                 float softmax_scale, int causal, int dtype, void *workspace,
                 int64_t workspace_bytes, rgd_cache *cache, void *stream);

/* rgd_attn_bwd plus the gradient of the additive bias, which the reference
 * refuses (flash_attn_triton_cached.py:1107).  `dbias` (null or kind
 * RGD_BIAS_NONE: exactly rgd_attn_bwd) describes the output and must have the
 * kind of `bias`:
 *   RGD_BIAS_VECTOR: dense fp32 [B, H, Tk] (dtype RGD_F32, stride_h = Tk,
 *     stride_b = H * Tk): sum over the queries of P * (dP - delta); zeroed by
 *     this call.
 *   RGD_BIAS_MATRIX: [B, H, Tq, Tk] in the q dtype through element strides
 *     (unit key stride): P * (dP - delta), one rounding.  With causal != 0 the
 *     entries of key blocks that lie entirely above the diagonal are NOT
 *     written: pass a zeroed tensor then.
 * The output always has full batch and head extents; a caller whose bias is
 * broadcast over batch, heads or queries sums over those dimensions. */
int rgd_attn_bwd_dbias(const rgd_heads *q, const rgd_heads *k,
                       const rgd_heads *v, const rgd_bias *bias,
                       const rgd_heads *o, const float *lse,
                       const rgd_heads *d_o, const rgd_heads *dq,
                       const rgd_heads *dk, const rgd_heads *dv,
                       const rgd_bias *dbias, int64_t B, int64_t H, int64_t Tq,
                       int64_t Tk, int64_t d, float softmax_scale, int causal,
                       int dtype, void *workspace, int64_t workspace_bytes,
                       rgd_cache *cache, void *stream);

/* Which attention implementation rgd_attn_fwd / rgd_attn_bwd take for these
 * views: 1 = tcgen05 / tensor-memory / TMA kernels, 0 = general mma.sync
 * kernels.  Evaluates exactly the test the entry points use (head_dim 64 or
 * 128, every view 16-byte addressable with positive strides on dimensions of
 * extent > 1, and for the forward softmax_scale > 0). */
int rgd_attn_fwd_uses_tmem(const rgd_heads *q, const rgd_heads *k,
                           const rgd_heads *v, const rgd_heads *o, int64_t B,
                           int64_t H, int64_t Tq, int64_t Tk, int64_t d,
                           float softmax_scale, int dtype);
int rgd_attn_bwd_uses_tmem(const rgd_heads *q, const rgd_heads *k,
                           const rgd_heads *v, const rgd_heads *o,
                           const rgd_heads *d_o, const rgd_heads *dq,
                           const rgd_heads *dk, const rgd_heads *dv, int64_t B,
                           int64_t H, int64_t Tq, int64_t Tk, int64_t d,
                           int dtype);

#ifdef __cplusplus
}
#endif
#endif /* RGD_B200_H */
