// Embedding gather with learned positions, and LayerNorm.
//
// embed:      x[t,:] = wte[token[t],:] (+ wpe[position[t],:])          -> float32 residual stream
//             (reference: include/model/ops.hpp:615-626, include/model/transformer.hpp:350-361);
//             optionally also the rows' statistics per 32-column segment (sum, squared deviation from the
//             segment's mean), which a product with a fused LayerNorm then uses instead of reading rows whole
// layernorm:  y = (x-mean) * 1/sqrt(var+eps) * gamma + beta, two passes over the row held in
//             shared memory, statistics in float32, biased variance
//             (reference: include/model/ops.hpp:443-476)
#include "common.cuh"

template <typename WT>
__global__ void embed_pos_kernel(const WT* __restrict__ wte, const WT* __restrict__ wpe,
                                 const int* __restrict__ tokens, const int* __restrict__ positions,
                                 float* __restrict__ x, int d, int V, int P, float* __restrict__ stats,
                                 int* __restrict__ dev_err) {
    const int t = blockIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    int tok = tokens[t];
    if (tok < 0 || tok >= V) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_TOKEN_RANGE);
        tok = min(max(tok, 0), V - 1);
    }
    const WT* e = wte + (size_t)tok * d;
    float* out = x + (size_t)t * d;
    const WT* p = nullptr;
    if (wpe != nullptr) {
        int pos = positions[t];
        if (pos < 0 || pos >= P) {
            if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_POSITION_RANGE);
            pos = min(max(pos, 0), P - 1);
        }
        p = wpe + (size_t)pos * d;
    }
    // a warp takes 32 consecutive columns at a time: one segment of the statistics
    const int lane = threadIdx.x & 31;
    for (int base = (threadIdx.x >> 5) * 32; base < d; base += blockDim.x) {
        const int i = base + lane;
        float v = 0.f;
        if (i < d) {
            v = ElemIO<WT>::load(e + i) + (p != nullptr ? ElemIO<WT>::load(p + i) : 0.f);
            out[i] = v;
        }
        if (stats != nullptr) {
            const float sum = warp_sum(v);
            const float dev = i < d ? v - sum / (float)min(32, d - base) : 0.f;
            const float m2 = warp_sum(dev * dev);
            if (lane == 0) {
                float* so = stats + ((size_t)t * ((d + 31) >> 5) + (base >> 5)) * 2;
                so[0] = sum; so[1] = m2;
            }
        }
    }
}

extern "C" int vlrf_embed(const void* wte, const void* wpe, int w_dtype, const int* tokens,
                          const int* positions, float* x, int T, int d, int V, int P,
                          float* stats /* or null: [T][ceil(d/32)][2] */, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && d > 0 && V > 0, "embed: bad sizes T=%d d=%d V=%d", T, d, V);
    VLRF_REQUIRE(wpe == nullptr || (positions != nullptr && P > 0), "embed: a position table needs positions");
    VLRF_REQUIRE(dev_err != nullptr, "embed: needs the device error word");
    if (T == 0) return VLRF_OK;
    const int threads = d >= 256 ? 256 : 128;
    if (w_dtype == VLRF_F32)
        launch_chained(embed_pos_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)wte, (const float*)wpe,
                       tokens, positions, x, d, V, P, stats, dev_err);
    else if (w_dtype == VLRF_BF16)
        launch_chained(embed_pos_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, (const __nv_bfloat16*)wte,
                       (const __nv_bfloat16*)wpe, tokens, positions, x, d, V, P, stats, dev_err);
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
    pdl_wait();
    pdl_launch_dependents();
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

// One warp per row, 16 bytes a lane a load; the row stays in registers when it has at most 2,048 values,
// else it is read a second and third time (from L1/L2).  For widths that are multiples of 4.
template <typename OT>
__global__ void __launch_bounds__(256) layernorm_warp_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                                              const float* __restrict__ gamma,
                                                              const float* __restrict__ beta, OT* __restrict__ out,
                                                              int n_rows, int d, float eps) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    pdl_wait();
    pdl_launch_dependents();
    if (r >= n_rows) return;
    const float4* src = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * d);
    const int nv = d >> 2;                       // float4s in the row
    constexpr int CACHE = 16;                    // float4s a lane keeps (16 × 32 × 4 = 2,048 values)
    float4 v[CACHE];
    const bool cached = nv <= CACHE * 32;
    float s = 0.f;
    if (cached) {
#pragma unroll
        for (int j = 0; j < CACHE; ++j) {
            const int i = j * 32 + lane;
            if (i < nv) { v[j] = src[i]; s += (v[j].x + v[j].y) + (v[j].z + v[j].w); }
        }
    } else {
        for (int i = lane; i < nv; i += 32) { const float4 a = src[i]; s += (a.x + a.y) + (a.z + a.w); }
    }
    const float mean = warp_sum(s) / (float)d;
    float q = 0.f;
    if (cached) {
#pragma unroll
        for (int j = 0; j < CACHE; ++j) {
            const int i = j * 32 + lane;
            if (i < nv) {
                const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, e = v[j].w - mean;
                q += (a * a + b * b) + (c * c + e * e);
            }
        }
    } else {
        for (int i = lane; i < nv; i += 32) {
            const float4 t = src[i];
            const float a = t.x - mean, b = t.y - mean, c = t.z - mean, e = t.w - mean;
            q += (a * a + b * b) + (c * c + e * e);
        }
    }
    const float inv = 1.f / sqrtf(warp_sum(q) / (float)d + eps);
    OT* dst = out + (size_t)r * d;
    const float4* g4 = reinterpret_cast<const float4*>(gamma);
    const float4* b4 = reinterpret_cast<const float4*>(beta);
    auto emit = [&](int i, const float4& t) {
        const float4 gm = g4[i], bt = b4[i];
        const float y0 = (t.x - mean) * inv * gm.x + bt.x, y1 = (t.y - mean) * inv * gm.y + bt.y;
        const float y2 = (t.z - mean) * inv * gm.z + bt.z, y3 = (t.w - mean) * inv * gm.w + bt.w;
        if (sizeof(OT) == 4) {
            reinterpret_cast<float4*>(dst)[i] = make_float4(y0, y1, y2, y3);
        } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            reinterpret_cast<uint2*>(dst)[i] = pk;
        }
    };
    if (cached) {
#pragma unroll
        for (int j = 0; j < CACHE; ++j) {
            const int i = j * 32 + lane;
            if (i < nv) emit(i, v[j]);
        }
    } else {
        for (int i = lane; i < nv; i += 32) emit(i, src[i]);
    }
}

// One warp per row of at most NV·128 values.  The norm's weight and bias do not depend on the kernel ahead:
// the CTA copies them to shared memory before the wait on it.  The row is read once and stays in registers.
template <typename OT, int NV>
__global__ void __launch_bounds__(256) layernorm_warp_small_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                                                    const float* __restrict__ gamma,
                                                                    const float* __restrict__ beta, OT* __restrict__ out,
                                                                    int n_rows, int d, float eps) {
    __shared__ float4 s_gamma[NV * 32], s_beta[NV * 32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    const int nv = d >> 2;
    for (int i = threadIdx.x; i < nv; i += 256) {
        s_gamma[i] = reinterpret_cast<const float4*>(gamma)[i];
        s_beta[i] = reinterpret_cast<const float4*>(beta)[i];
    }
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    if (r >= n_rows) return;
    const float* src = x + (size_t)(rows ? rows[r] : r) * d;
    float4 v[NV];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = j * 32 + lane;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < nv)      // an explicit load: the values stay in registers for all three passes
            asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];"
                         : "=f"(v[j].x), "=f"(v[j].y), "=f"(v[j].z), "=f"(v[j].w) : "l"(src + 4 * i));
        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
    }
    const float mean = warp_sum(s) / (float)d;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
        if (j * 32 + lane < nv) {
            const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, e = v[j].w - mean;
            q += (a * a + b * b) + (c * c + e * e);
        }
    const float inv = 1.f / sqrtf(warp_sum(q) / (float)d + eps);
    OT* dst = out + (size_t)r * d;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int i = j * 32 + lane;
        if (i < nv) {
            const float4 gm = s_gamma[i], bt = s_beta[i];
            const float y0 = (v[j].x - mean) * inv * gm.x + bt.x, y1 = (v[j].y - mean) * inv * gm.y + bt.y;
            const float y2 = (v[j].z - mean) * inv * gm.z + bt.z, y3 = (v[j].w - mean) * inv * gm.w + bt.w;
            if (sizeof(OT) == 4) {
                reinterpret_cast<float4*>(dst)[i] = make_float4(y0, y1, y2, y3);
            } else {
                __nv_bfloat162 lo = __floats2bfloat162_rn(y0, y1), hi = __floats2bfloat162_rn(y2, y3);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo);
                pk.y = *reinterpret_cast<uint32_t*>(&hi);
                reinterpret_cast<uint2*>(dst)[i] = pk;
            }
        }
    }
}

extern "C" int vlrf_layernorm(const float* x, const int* rows, const float* gamma, const float* beta,
                              void* out, int out_dtype, int n_rows, int d, float eps,
                              cudaStream_t stream) {
    VLRF_REQUIRE(n_rows >= 0 && d > 0, "layernorm: bad sizes rows=%d d=%d", n_rows, d);
    VLRF_REQUIRE(d <= 48 * 1024 / 4 - 32, "layernorm: width %d exceeds the %d this kernel holds in shared memory",
                 d, 48 * 1024 / 4 - 32);
    if (n_rows == 0) return VLRF_OK;
    if (d % 4 == 0 && n_rows >= 8) {
        const dim3 grid((n_rows + 7) / 8);
        if (d <= 1024 && out_dtype == VLRF_F32)
            launch_chained(layernorm_warp_small_kernel<float, 8>, grid, dim3(256), 0, stream, x, rows, gamma, beta, (float*)out, n_rows, d, eps);
        else if (d <= 1024 && out_dtype == VLRF_BF16)
            launch_chained(layernorm_warp_small_kernel<__nv_bfloat16, 8>, grid, dim3(256), 0, stream, x, rows, gamma, beta,
                           (__nv_bfloat16*)out, n_rows, d, eps);
        else if (d <= 2048 && out_dtype == VLRF_F32)
            launch_chained(layernorm_warp_small_kernel<float, 16>, grid, dim3(256), 0, stream, x, rows, gamma, beta, (float*)out, n_rows, d, eps);
        else if (d <= 2048 && out_dtype == VLRF_BF16)
            launch_chained(layernorm_warp_small_kernel<__nv_bfloat16, 16>, grid, dim3(256), 0, stream, x, rows, gamma, beta,
                           (__nv_bfloat16*)out, n_rows, d, eps);
        else if (out_dtype == VLRF_F32)
            launch_chained(layernorm_warp_kernel<float>, grid, dim3(256), 0, stream, x, rows, gamma, beta, (float*)out, n_rows, d, eps);
        else if (out_dtype == VLRF_BF16)
            launch_chained(layernorm_warp_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, x, rows, gamma, beta,
                           (__nv_bfloat16*)out, n_rows, d, eps);
        else
            return vlrf_fail(VLRF_ERR_INVALID_ARG, "layernorm: unknown output dtype %d", out_dtype);
        return vlrf_check_launch("layernorm");
    }
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
