// Host helpers for the tensor-memory kernels: TMA tensor-map encoding through
// the driver entry point (no link-time dependency on libcuda) and the sticky
// device status word.
#include <mutex>
#include <new>
#include <string.h>
#include <vector>

#include "sm100_prims.cuh"

// A launch-plan cache: the tensor-map descriptors of the attention calls it has seen, keyed on
// everything that goes into a descriptor (base pointer, extents, strides, box, element type).
// A call whose tensors moved or changed shape simply misses and encodes afresh, so a stale
// entry can never be launched with.  Entries are few (a training step reuses the same handful
// of buffers), so a small array with round-robin replacement is enough.
struct rgd_cache {
    struct Entry {
        const void *base;
        int64_t v[10];           // B, H, T, d, stride_b, stride_h, stride_n, box_d, box_t, bf16
        CUtensorMap map;
    };
    static constexpr size_t CAPACITY = 64;
    std::mutex mu;
    std::vector<Entry> entries;
    size_t next = 0;
    int64_t hits = 0, misses = 0;
};

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

bool heads_map_encodable(const void *base, int64_t B, int64_t H, int64_t T, int64_t stride_b, int64_t stride_h,
                         int64_t stride_n) {
    if (!is_aligned(base, 16)) return false;
    const int64_t limit = (1ll << 40) / 2;      // descriptor strides are below 2^40 bytes
    auto ok = [&](int64_t extent, int64_t stride) {
        return extent <= 1 || (stride > 0 && stride % 8 == 0 && stride < limit);
    };
    return ok(T, stride_n) && ok(H, stride_h) && ok(B, stride_b);
}

int encode_heads_map_cached(rgd_cache *cache, CUtensorMap *out, const void *base, int64_t B, int64_t H, int64_t T,
                            int64_t d, int64_t stride_b, int64_t stride_h, int64_t stride_n, int box_d, int box_t,
                            bool bf16) {
    if (!cache) return encode_heads_map(out, base, B, H, T, d, stride_b, stride_h, stride_n, box_d, box_t, bf16);
    const int64_t v[10] = {B, H, T, d, stride_b, stride_h, stride_n, box_d, box_t, bf16 ? 1 : 0};
    std::lock_guard<std::mutex> lock(cache->mu);
    for (const rgd_cache::Entry &e : cache->entries)
        if (e.base == base && memcmp(e.v, v, sizeof(v)) == 0) {
            *out = e.map;
            ++cache->hits;
            return RGD_OK;
        }
    ++cache->misses;
    if (int rc = encode_heads_map(out, base, B, H, T, d, stride_b, stride_h, stride_n, box_d, box_t, bf16)) return rc;
    rgd_cache::Entry e;
    e.base = base;
    memcpy(e.v, v, sizeof(v));
    e.map = *out;
    if (cache->entries.size() < rgd_cache::CAPACITY) {
        cache->entries.push_back(e);
    } else {
        cache->entries[cache->next] = e;
        cache->next = (cache->next + 1) % rgd_cache::CAPACITY;
    }
    return RGD_OK;
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

extern "C" rgd_cache *rgd_cache_create(void) { return new (std::nothrow) rgd_cache(); }

extern "C" void rgd_cache_destroy(rgd_cache *cache) { delete cache; }

extern "C" int rgd_cache_stats(rgd_cache *cache, int64_t *hits, int64_t *misses, int64_t *entries) {
    if (!cache) return RGD_E_NULL;
    std::lock_guard<std::mutex> lock(cache->mu);
    if (hits) *hits = cache->hits;
    if (misses) *misses = cache->misses;
    if (entries) *entries = (int64_t)cache->entries.size();
    return RGD_OK;
}
