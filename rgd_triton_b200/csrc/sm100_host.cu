// Host helpers for the tensor-memory kernels: TMA tensor-map encoding through
// the driver entry point (no link-time dependency on libcuda) and the sticky
// device status word.
#include <mutex>

#include "sm100_prims.cuh"

namespace rgd {
namespace sm100 {

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encoder() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            (void)cudaGetLastError();
    });
    return fn;
}

int encode_heads_map(CUtensorMap *out, const void *base, int64_t B, int64_t H, int64_t T, int64_t d,
                     int64_t stride_b, int64_t stride_h, int64_t stride_n, int box_d, int box_t, bool bf16) {
    EncodeTiledFn fn = encoder();
    if (!fn) return RGD_E_DEVICE;
    if (!is_aligned(base, 16)) return RGD_E_STRIDE;
    // A dimension of extent 1 never advances: give it any legal stride.
    const int64_t row_bytes = d * 2;
    int64_t sn = stride_n * 2, sh = stride_h * 2, sb = stride_b * 2;
    if (T == 1) sn = row_bytes;
    if (H == 1) sh = row_bytes;
    if (B == 1) sb = row_bytes;
    if (sn % 16 || sh % 16 || sb % 16 || sn <= 0 || sh <= 0 || sb <= 0) return RGD_E_STRIDE;
    cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)sn, (cuuint64_t)sh, (cuuint64_t)sb};
    cuuint32_t box[4] = {(cuuint32_t)box_d, (cuuint32_t)box_t, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? RGD_OK : RGD_E_STRIDE;
}

}  // namespace sm100
}  // namespace rgd
