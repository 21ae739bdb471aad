// Host-side helpers of the sm_100a kernels: tensor-map creation and device facts.
#include "sm100_ptx.cuh"
#include <mutex>
#include <unordered_map>

TiEncodeTiledFn ti_encode_tiled_fn() {
    static TiEncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<TiEncodeTiledFn>(ptr);
    });
    return fn;
}

namespace {
struct MapKey {
    const void* ptr; long long rows; int k, box_rows;
    bool operator==(const MapKey& o) const { return ptr == o.ptr && rows == o.rows && k == o.k && box_rows == o.box_rows; }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ (size_t)k.rows * 1000003u ^ (size_t)k.k * 10007u ^ (size_t)k.box_rows;
    }
};

}  // namespace

// A tensor map of a row-major [rows, k] bf16 matrix, boxes of box_rows x 64, 128-byte swizzle.
bool ti_get_bf16_map(const void* ptr, long long rows, int k, int box_rows, CUtensorMap* out) {
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    const MapKey key{ptr, rows, k, box_rows};
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    TiEncodeTiledFn fn = ti_encode_tiled_fn();
    if (!fn) { ti_set_error("cuTensorMapEncodeTiled is not available from this driver"); return false; }
    cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)k * 2};
    cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { ti_set_error("cuTensorMapEncodeTiled failed (%d) for [%lld, %d] box %d", (int)r, rows, k, box_rows); return false; }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

int ti_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    }
    return n;
}

