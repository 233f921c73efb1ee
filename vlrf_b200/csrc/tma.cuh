// Tensor-map (TMA) helpers: encoding 2-D bfloat16 tensor maps on the host through the driver entry point
// fetched at run time (nothing links against libcuda), and the device-side load.
//
// A tiled TMA load must start on a 16-byte boundary in the innermost dimension: callers pass x as a
// multiple of 8 elements.  Coordinates outside the tensor read zeros, so ragged edges need no special
// case.  No load here uses cluster multicast.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>

// rows × cols bfloat16, row stride `ld` elements, box of box_rows × box_cols elements, 128-byte swizzle
// (box_cols·2 must be 128).  Returns 0 and fills `out`, or a status with vlrf_last_error() set.
int vlrf_make_tmap_bf16(const void* ptr, long long rows, long long cols, long long ld, int box_rows, int box_cols,
                        CUtensorMap* out);

__device__ __forceinline__ uint32_t tma_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tmap, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(tma_smem_u32(dst)), "l"(tmap), "r"(tma_smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
