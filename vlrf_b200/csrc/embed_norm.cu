// Embedding gather with learned positions, and LayerNorm.
//
// embed:      x[t,:] = wte[token[t],:] (+ wpe[position[t],:])          -> float32 residual stream
//             (reference: include/model/ops.hpp:615-626, include/model/transformer.hpp:350-361)
// layernorm:  y = (x-mean) * 1/sqrt(var+eps) * gamma + beta, two passes over the row held in
//             shared memory, statistics in float32, biased variance
//             (reference: include/model/ops.hpp:443-476)
#include "common.cuh"

template <typename WT>
__global__ void embed_pos_kernel(const WT* __restrict__ wte, const WT* __restrict__ wpe,
                                 const int* __restrict__ tokens, const int* __restrict__ positions,
                                 float* __restrict__ x, int d, int V, int P, int* __restrict__ dev_err) {
    const int t = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    int tok = tokens[t];
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_TOKEN_RANGE);
        tok = min(max(tok, 0), V - 1);
    }
    const WT* e = wte + (size_t)tok * d;
    float* out = x + (size_t)t * d;
    if (wpe != nullptr) {
        int pos = positions[t];
        if (pos < 0 || pos >= P) {
            if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_POSITION_RANGE);
            pos = min(max(pos, 0), P - 1);
        }
        const WT* p = wpe + (size_t)pos * d;
        for (int i = threadIdx.x; i < d; i += blockDim.x)
            out[i] = ElemIO<WT>::load(e + i) + ElemIO<WT>::load(p + i);
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = ElemIO<WT>::load(e + i);
    }
}

extern "C" int vlrf_embed(const void* wte, const void* wpe, int w_dtype, const int* tokens,
                          const int* positions, float* x, int T, int d, int V, int P, int* dev_err,
                          cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && d > 0 && V > 0, "embed: bad sizes T=%d d=%d V=%d", T, d, V);
    VLRF_REQUIRE(wpe == nullptr || (positions != nullptr && P > 0), "embed: a position table needs positions");
    VLRF_REQUIRE(dev_err != nullptr, "embed: needs the device error word");
    if (T == 0) return VLRF_OK;
    const int threads = d >= 256 ? 256 : 128;
    if (w_dtype == VLRF_F32)
        launch_chained(embed_pos_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)wte, (const float*)wpe,
                       tokens, positions, x, d, V, P, dev_err);
    else if (w_dtype == VLRF_BF16)
        launch_chained(embed_pos_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)wte,
                       (const __nv_bfloat16*)wpe, tokens, positions, x, d, V, P, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "embed: unknown weight dtype %d", w_dtype);
    return vlrf_check_launch("embed");
}

// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ float block_sum(float v, float* red) {
    // red: one float per warp, in shared memory
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();  // protect `red` from the previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarp; ++w) total += red[w];  // same order in every thread
    return total;
}

template <typename OT>
__global__ void layernorm_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                 const float* __restrict__ gamma, const float* __restrict__ beta,
                                 OT* __restrict__ out, int d, float eps) {
    extern __shared__ float smem[];
    float* row = smem;          // d floats
    float* red = smem + d;      // 32 floats
    const int r = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    const float* src = x + (size_t)(rows ? rows[r] : r) * d;
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = src[i];
        row[i] = v;
        s += v;
    }
    const float mean = block_sum(s, red) / (float)d;
    float q = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float c = row[i] - mean;
        q += c * c;
    }
    const float var = block_sum(q, red) / (float)d + eps;
    const float inv = 1.f / sqrtf(var);
    OT* dst = out + (size_t)r * d;
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        ElemIO<OT>::store(dst + i, (row[i] - mean) * inv * gamma[i] + beta[i]);
}

extern "C" int vlrf_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                              void* out, int out_dtype, int n_rows, int d, float eps,
                              cudaStream_t stream) {
    VLRF_REQUIRE(n_rows >= 0 && d > 0, "layernorm: bad sizes rows=%d d=%d", n_rows, d);
    VLRF_REQUIRE(d <= 48 * 1024 / 4 - 32, "layernorm: width %d exceeds the %d this kernel holds in shared memory",
                 d, 48 * 1024 / 4 - 32);
    if (n_rows == 0) return VLRF_OK;
    const int threads = d >= 1024 ? 256 : 128;
    const size_t smem = (size_t)(d + 32) * sizeof(float);
    if (out_dtype == VLRF_F32)
        launch_chained(layernorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta, (float*)out, d, eps);
    else if (out_dtype == VLRF_BF16)
        launch_chained(layernorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), smem, stream, x, rows, gamma, beta,
                       (__nv_bfloat16*)out, d, eps);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "layernorm: unknown output dtype %d", out_dtype);
    return vlrf_check_launch("layernorm");
}
