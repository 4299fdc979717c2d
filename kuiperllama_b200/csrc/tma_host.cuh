// Host side of TMA: building (and keeping) tensor maps over bfloat16 tensors.  The driver's
// cuTensorMapEncodeTiled is fetched through the runtime (cudaGetDriverEntryPoint), so the
// libraries do not link against libcuda.
#pragma once
#include "common.cuh"
#include <cuda.h>
#include <stdio.h>
#include <mutex>
#include <unordered_map>

namespace kl {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tma_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

struct TmaKey {
    const void* ptr;
    int rank;
    long long dims[3], strides[2];
    int box[3];
    bool operator==(const TmaKey& o) const { return memcmp(this, &o, sizeof(TmaKey)) == 0; }
};
struct TmaKeyHash {
    size_t operator()(const TmaKey& k) const {
        const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
        size_t h = 1469598103934665603ull;
        for (size_t i = 0; i < sizeof(TmaKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
        return h;
    }
};

// A map over a bfloat16 tensor of `rank` dimensions (innermost first): dims in elements,
// strides of dimensions 1.. in elements (dimension 0 is contiguous), box in elements; 128-byte
// swizzle (the box's innermost extent must be 64 elements), zero fill outside the tensor.
// Maps are kept: weights and caches come back with the same address every step.
inline int tma_make_map(CUtensorMap* out, const void* ptr, int rank, const long long* dims, const long long* strides,
                        const int* box) {
    static std::unordered_map<TmaKey, CUtensorMap, TmaKeyHash> cache;
    static std::mutex mu;
    TmaKey key;
    memset(&key, 0, sizeof(key));
    key.ptr = ptr;
    key.rank = rank;
    for (int i = 0; i < rank; ++i) { key.dims[i] = dims[i]; key.box[i] = box[i]; }
    for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides[i];
    {
        std::lock_guard<std::mutex> g(mu);
        auto it = cache.find(key);
        if (it != cache.end()) { *out = it->second; return KL_OK; }
    }
    EncodeTiledFn fn = tma_encode_fn();
    if (!fn) return KL_ERR_SETUP;
    cuuint64_t d[3], s[2];
    cuuint32_t b[3], e[3] = {1, 1, 1};
    for (int i = 0; i < rank; ++i) { d[i] = (cuuint64_t)dims[i]; b[i] = (cuuint32_t)box[i]; }
    for (int i = 0; i + 1 < rank; ++i) s[i] = (cuuint64_t)strides[i] * 2;
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(ptr), d, s, b, e,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        fprintf(stderr, "[kuiperllama_b200] cuTensorMapEncodeTiled failed with %d (rank %d, dims %lld %lld %lld, box %d %d %d)\n",
                (int)r, rank, key.dims[0], key.dims[1], key.dims[2], key.box[0], key.box[1], key.box[2]);
        return KL_ERR_SETUP;
    }
    std::lock_guard<std::mutex> g(mu);
    if (cache.size() > 4096) cache.clear();
    cache[key] = *out;
    return KL_OK;
}

}  // namespace kl
