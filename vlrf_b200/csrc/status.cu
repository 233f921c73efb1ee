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
