// TMA tensor maps through the driver entry point (no link against libcuda), cached by what defines them.
#include "tensor_map.h"

#include "common.cuh"

#include <cstring>
#include <mutex>
#include <unordered_map>

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

struct MapKey {
    const void* ptr;
    unsigned long long dims[3], strides[2];
    unsigned box[3];
    int rank, swizzle;
    bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapHash {
    size_t operator()(const MapKey& k) const {
        size_t h = (size_t)k.ptr;
        for (int i = 0; i < 3; ++i) h = (h * 1000003u ^ (size_t)k.dims[i]) * 1000003u ^ (size_t)k.box[i];
        for (int i = 0; i < 2; ++i) h = h * 1000003u ^ (size_t)k.strides[i];
        return (h * 1000003u ^ (size_t)k.rank) * 1000003u ^ (size_t)k.swizzle;
    }
};

}  // namespace

int ti_tensor_map_bf16(CUtensorMap* out, const void* ptr, int rank, const unsigned long long* dims,
                       const unsigned long long* strides, const unsigned* box, bool swizzle128) {
    static std::unordered_map<MapKey, CUtensorMap, MapHash> cache;
    static std::mutex mu;
    TI_REQUIRE(rank == 2 || rank == 3, "tensor map: rank %d", rank);
    MapKey key;
    std::memset(&key, 0, sizeof(key));                   // padding bytes too: keys are compared as bytes
    key.ptr = ptr; key.rank = rank; key.swizzle = swizzle128 ? 1 : 0;
    for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
    std::lock_guard<std::mutex> lock(mu);
    auto hit = cache.find(key);
    if (hit != cache.end()) { *out = hit->second; return 0; }
    EncodeTiledFn enc = encode_fn();
    if (!enc) return ti_fail("tensor map: cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t d[3], s[2];
    cuuint32_t b[3], e[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; b[i] = box[i]; }
    for (int i = 0; i + 1 < rank; ++i) s[i] = strides[i];
    CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), d, s, b, e,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ti_fail("tensor map: cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, *out);
    return 0;
}
