// Shared declarations of the sm_100a kernels: status codes, the last-error
// string, element types and small device helpers.  Every exported function is
// `extern "C"`, takes raw device pointers and the stream to launch on, checks
// its sizes on the host before launching anything, and returns 0 or a status
// whose text `vlrf_last_error()` gives.  Nothing here allocates device memory.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <cstdio>
#include <cstdarg>

// Status codes (same numbering idea as the reference's status enum, include/api/vlrf.h:32-41), element types,
// activations, the bits of the device-side error word that kernels set instead of faulting, and the prototype of
// every exported function: the definitions in the .cu files are checked against them by the compiler.
#include "vlrf_b200_kernels.h"

extern "C" const char* vlrf_last_error();
int vlrf_fail(int code, const char* fmt, ...);
int vlrf_check_launch(const char* what);

#define VLRF_REQUIRE(cond, ...) \
    do { if (!(cond)) return vlrf_fail(VLRF_ERR_INVALID_ARG, __VA_ARGS__); } while (0)

// Programmatic dependent launch: a kernel launched through `launch_chained` may begin while the kernel
// before it on the stream is still running.  It may do only what does not depend on that kernel (set up
// shared memory, start fetching weights) until `pdl_wait()` returns, which happens once every earlier
// kernel has finished and its writes are visible.  `pdl_launch_dependents()` lets the next kernel begin in
// the same way.  Every kernel of the step calls both.  The products, which read nothing but weights before
// their wait, release their successor at once; every other kernel only after its own wait.  So when a
// kernel begins, at least one kernel that is not a product lies complete between it and whatever wrote the
// positions, the block tables and the cache of earlier positions (the sampling kernel of the step before,
// host copies, the step before's projections): decode attention may fetch those before its wait, but
// nothing that the kernels just ahead write (activations, the new position's key and value).
// `vlrf_set_chained_launch(0)` turns the launch attribute off (the calls then do nothing).
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
extern "C" int vlrf_chained_launch_enabled();

// Time stamps inside the kernels of a decode step, compiled in only with -DVLRF_KERNEL_TRACE (build.py:
// VLRF_B200_KERNEL_TRACE=1).  One thread of a CTA calls VLRF_TRACE(buf, kind, cta, station) at the stations of the
// kernel's critical path; the record of a launch is found by the launch's number (%gridid), so a replayed graph
// leaves the stamps of its last replay.  buf: [VLRF_TRACE_SLOTS][VLRF_TRACE_CTAS][2 + VLRF_TRACE_STATIONS] int64:
// launch number, kind of kernel, then nanoseconds of the global timer (coarse: steps of a quarter microsecond).
constexpr int VLRF_TRACE_SLOTS = 512, VLRF_TRACE_CTAS = 512, VLRF_TRACE_STATIONS = 8;
extern "C" long long* vlrf_trace_buffer();     // device memory, or null in a build without stamps
#ifdef VLRF_KERNEL_TRACE
__device__ __forceinline__ void vlrf_trace_stamp(long long* buf, int kind, int cta, int station) {
    unsigned long long gid;
    long long t;
    asm volatile("mov.u64 %0, %%gridid;" : "=l"(gid));
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (buf != nullptr && cta < VLRF_TRACE_CTAS) {
        long long* r = buf + ((size_t)(gid % VLRF_TRACE_SLOTS) * VLRF_TRACE_CTAS + cta) * (2 + VLRF_TRACE_STATIONS);
        r[0] = (long long)gid; r[1] = kind; r[2 + station] = t;
    }
}
#define VLRF_TRACE(buf, kind, cta, station) vlrf_trace_stamp(buf, kind, cta, station)
#else
#define VLRF_TRACE(buf, kind, cta, station) ((void)0)
#endif

template <typename... KArgs, typename... Args>
cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                           Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    // every kernel of a step asks for the same split of an SM's memory between shared memory and L1 (all of
    // it shared): an SM changes the split only when it is empty, which would keep kernels that want different
    // splits from running side by side
    attr[0].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
    attr[0].val.sharedMemCarveout = cudaSharedmemCarveoutMaxShared;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vlrf_chained_launch_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// The same for a kernel whose CTAs form clusters of the given shape: the CTAs of a cluster run at the same
// time on neighbouring SMs and may read one another's shared memory.
template <typename... KArgs, typename... Args>
cudaError_t launch_chained_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, dim3 cluster,
                                   cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[3];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster.x;
    attr[0].val.clusterDim.y = cluster.y;
    attr[0].val.clusterDim.z = cluster.z;
    attr[1].id = cudaLaunchAttributePreferredSharedMemoryCarveout;
    attr[1].val.sharedMemCarveout = cudaSharedmemCarveoutMaxShared;
    attr[2].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[2].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = vlrf_chained_launch_enabled() ? 3 : 2;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Thread-block clusters: a barrier of all threads of all CTAs of the cluster (with release/acquire ordering
// of memory, shared memory of the other CTAs included), and reading another CTA's shared memory.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the same without ordering of memory: for "everyone has finished reading", when what was read has been used
__device__ __forceinline__ void cluster_sync_relaxed() {
    asm volatile("barrier.cluster.arrive.relaxed.aligned;\nbarrier.cluster.wait.aligned;" ::: "memory");
}
// the value at `own_addr` (a shared-memory address of this CTA) in the CTA of rank `rank` of the cluster
__device__ __forceinline__ float ld_cluster_f32(uint32_t own_addr, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(own_addr), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}
// … and 16 bytes of it (own_addr a multiple of 16)
__device__ __forceinline__ float4 ld_cluster_f32x4(uint32_t own_addr, uint32_t rank) {
    uint32_t remote;
    float4 v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(own_addr), "r"(rank));
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote) : "memory");
    return v;
}

template <typename T> struct ElemIO;
template <> struct ElemIO<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct ElemIO<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// GELU as the reference computes it (tanh form, include/model/ops.hpp:390-403)
// and the exact erf form for activation_function "gelu".
__device__ __forceinline__ float gelu_tanh_f(float x) {
    const float c1 = 0.7978845608028654f, c2 = 0.044715f;
    return 0.5f * x * (1.f + tanhf(c1 * (x + c2 * x * x * x)));
}
__device__ __forceinline__ float gelu_erf_f(float x) {
    return 0.5f * x * (1.f + erff(x * 0.70710678118654752440f));
}
template <int ACT> __device__ __forceinline__ float apply_act(float x) {
    if (ACT == VLRF_ACT_GELU_TANH) return gelu_tanh_f(x);
    if (ACT == VLRF_ACT_GELU_ERF) return gelu_erf_f(x);
    return x;
}
// The tanh form for results that are rounded to bfloat16 anyway: tanh in one instruction (`tanh.approx.f32`,
// relative error about 2^-11, below bfloat16's 2^-9).  Every bfloat16-output epilogue uses this one, so a
// token's value does not depend on which product kernel its step took; float32 outputs keep tanhf.
__device__ __forceinline__ float gelu_tanh_fast(float x) {
    const float c1 = 0.7978845608028654f, c2 = 0.044715f;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(c1 * (x + c2 * x * x * x)));
    return 0.5f * x * (1.f + t);
}
template <typename OT> __device__ __forceinline__ float apply_act_out(float x, int act) {
    if (act == VLRF_ACT_GELU_TANH) return sizeof(OT) == 2 ? gelu_tanh_fast(x) : gelu_tanh_f(x);
    if (act == VLRF_ACT_GELU_ERF) return gelu_erf_f(x);
    return x;
}
// 32 bytes a thread in one instruction (sm_100): a thread that writes its own row piece by piece fills a whole
// 32-byte sector at a time this way; with 16-byte pieces every sector goes to L2 twice, half full
__device__ __forceinline__ void st_global_32B(void* p, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]),
                 "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}
__device__ __forceinline__ void ld_global_32B(const void* p, float (&v)[8]) {
    asm volatile("ld.global.v8.f32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];" : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]),
                 "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]) : "l"(p) : "memory");
}
// the same with the activation known at compile time (a run-time `act` per element costs issue slots: the
// branches become predicates, and the paths not taken are still issued)
template <typename OT, int ACT> __device__ __forceinline__ float apply_act_const(float x) {
    if (ACT == VLRF_ACT_GELU_TANH) return sizeof(OT) == 2 ? gelu_tanh_fast(x) : gelu_tanh_f(x);
    if (ACT == VLRF_ACT_GELU_ERF) return gelu_erf_f(x);
    return x;
}
__device__ __forceinline__ float apply_act_rt(float x, int act) {
    if (act == VLRF_ACT_GELU_TANH) return gelu_tanh_f(x);
    if (act == VLRF_ACT_GELU_ERF) return gelu_erf_f(x);
    return x;
}
