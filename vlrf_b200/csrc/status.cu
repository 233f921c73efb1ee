// The last-error string and launch checking shared by all kernels' host entry points.
#include "common.cuh"
#include <mutex>

static thread_local char g_last_error[512] = "";

extern "C" const char* vlrf_last_error() { return g_last_error; }

int vlrf_fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

int vlrf_check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    return VLRF_OK;
}

extern "C" int vlrf_device_info(int* sm_count, int* cc_major, int* cc_minor, int* max_smem_optin) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
    cudaDeviceProp p;
    e = cudaGetDeviceProperties(&p, dev);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
    *sm_count = p.multiProcessorCount;
    *cc_major = p.major;
    *cc_minor = p.minor;
    *max_smem_optin = (int)p.sharedMemPerBlockOptin;
    return VLRF_OK;
}

static int g_chained = 1;
extern "C" int vlrf_chained_launch_enabled() { return g_chained; }
extern "C" int vlrf_set_chained_launch(int on) { g_chained = on ? 1 : 0; return VLRF_OK; }

// The buffer of the kernels' time stamps (common.cuh): allocated at the first call in a build with stamps.
static long long* g_trace = nullptr;
extern "C" long long* vlrf_trace_buffer() {
#ifdef VLRF_KERNEL_TRACE
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
    if (g_trace == nullptr) {
        const size_t bytes = sizeof(long long) * VLRF_TRACE_SLOTS * VLRF_TRACE_CTAS * (2 + VLRF_TRACE_STATIONS);
        if (cudaMalloc(&g_trace, bytes) != cudaSuccess) { g_trace = nullptr; return nullptr; }
        cudaMemset(g_trace, 0, bytes);
    }
#endif
    return g_trace;
}
// slots, CTAs a slot and stations a CTA of the stamp buffer; 0 slots in a build without stamps
extern "C" int vlrf_trace_dims(int* slots, int* ctas, int* stations) {
#ifdef VLRF_KERNEL_TRACE
    *slots = VLRF_TRACE_SLOTS;
#else
    *slots = 0;
#endif
    *ctas = VLRF_TRACE_CTAS; *stations = VLRF_TRACE_STATIONS;
    return VLRF_OK;
}
// copies the stamps to `host` ([slots][ctas][2 + stations] int64) and clears them
extern "C" int vlrf_trace_read(long long* host) {
    long long* buf = vlrf_trace_buffer();
    if (buf == nullptr) return vlrf_fail(VLRF_ERR_INVALID_ARG, "this build has no time stamps (build with VLRF_B200_KERNEL_TRACE=1)");
    const size_t bytes = sizeof(long long) * VLRF_TRACE_SLOTS * VLRF_TRACE_CTAS * (2 + VLRF_TRACE_STATIONS);
    cudaError_t e = cudaMemcpy(host, buf, bytes, cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaMemset(buf, 0, bytes);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "trace: %s", cudaGetErrorString(e));
    return VLRF_OK;
}
