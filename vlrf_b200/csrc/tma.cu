// Host side of the tensor-map helpers: cuTensorMapEncodeTiled through cudaGetDriverEntryPoint, with a
// cache so that a weight's map is encoded once.
#include "common.cuh"
#include "tma.cuh"
#include <map>
#include <mutex>
#include <tuple>

namespace {
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::mutex g_mutex;
typedef std::tuple<const void*, long long, long long, long long, int, int> Key;
std::map<Key, CUtensorMap> g_cache;
}  // namespace

int vlrf_make_tmap_bf16(const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols,
                        CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_mutex);
    const Key key(ptr, rows, cols, ld, box_rows, box_cols);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) { *out = it->second; return VLRF_OK; }
    if (g_encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
        if (e != cudaSuccess || fn == nullptr || qres != cudaDriverEntryPointSuccess)
            return vlrf_fail(VLRF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || (ld * 2) % 16 != 0)
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "tensor map: base and row stride must be multiples of 16 bytes (ld=%lld)", ld);
    if (box_cols * 2 != 128 || box_rows < 1 || box_rows > 256)
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "tensor map: box %d x %d is not 1…256 rows of 128 bytes", box_rows, box_cols);
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t elem[2] = {1, 1};
    CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return vlrf_fail(VLRF_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (g_cache.size() > 4096) g_cache.clear();   // activations' buffers come and go; weights re-enter on next use
    g_cache[key] = *out;
    return VLRF_OK;
}
