// Y[M,N] = act(X[M,K] · W[N,K]^T + bias) (+ residual) for few rows (M ≤ 64): the decode step's products.
//
// With a handful of rows the product is bound by reading W once, so the kernel is built to stream W:
// the weight's rows are the 16-row operand of `mma.sync.m16n8k16` (bf16 in, float32 accumulate) and
// the batch rows are the 8-column operand, eight at a time.  A warp owns 16 output columns and a share
// of K; every lane fetches 16 contiguous bytes of a weight row per load, several loads in flight, and
// because a sum over k may run in any order the 8 values of one load are fed to two MMAs directly — no
// shared-memory staging of W.  The warps that share a column group add their partial sums in a fixed
// order, so the result does not depend on timing.
//
// Fusions: LayerNorm of the float32 residual rows in the prologue (statistics in float32, two passes,
// reference include/model/ops.hpp:443-476), bias / GELU / residual sum in the epilogue (reference
// include/model/feedforward.hpp:54-76, include/model/transformer_block.hpp:153,158), and the scatter of
// the K and V columns of a fused q/k/v projection into the paged cache (reference
// include/model/kv_cache.hpp:215-251).
#include "common.cuh"

namespace {

constexpr int SK_THREADS = 512;
constexpr int SK_WARPS = 16;
// 32-wide k-chunks a warp has in flight at once (two 16-byte loads per lane each); fewer when many batch
// tiles need the registers
template <int MT> struct Unroll { static constexpr int value = MT <= 2 ? 8 : (MT == 4 ? 4 : 2); };

struct KvScatter {
    void* Kc; void* Vc;            // this layer's cache [block][kv_head][BT][dh], bf16
    const int* block_table; const int* tok_slot; const int* tok_pos;
    int max_blocks, k_off, v_off, width, dh, Hkv, BT;   // width = Hkv*dh
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
// weights are read once: keep them from pushing the activations out of L1
__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// MT: number of 8-row tiles of the batch; LN: X is float32 [M,K] to be normalised, else bf16 [M,K]
template <int MT, bool LN, typename OT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const void* __restrict__ Xv, const __nv_bfloat16* __restrict__ W,
                   const float* __restrict__ bias, const float* residual, OT* Y, int M, int N, int K, int ldx,
                   int ldy, int act, int ksplit, const float* __restrict__ gamma,
                   const float* __restrict__ beta, float eps, KvScatter kv) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int groups_per_cta = SK_WARPS / ksplit;
    const int group = warp / ksplit, kpart = warp % ksplit;
    const int n0 = (blockIdx.x * groups_per_cta + group) * 16;

    // shared memory: [LN: normalised X as bf16, row stride xs_stride bytes][partials for the k-split]
    const int xs_stride = LN ? (K * 2 + 64 + ((128 - (K * 2) % 128) % 128)) : 0;   // ≡ 64 mod 128: conflict-free
    unsigned char* xs = smem_raw;
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)xs_stride * MT * 8);

    constexpr int UNROLL = Unroll<MT>::value;
    if (LN) {
        const float* X = reinterpret_cast<const float*>(Xv);
        const bool cached = (K % 128 == 0) && K <= 1024 && (ldx % 4 == 0);
        for (int m = warp; m < MT * 8; m += SK_WARPS) {
            const float* row = X + (size_t)min(m, M - 1) * ldx;
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(xs + (size_t)m * xs_stride);
            if (cached) {
                // the row is read once, 16 bytes a lane a load, and stays in registers for both passes
                float4 v[8];
                const int nv = K / 128;
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < nv) {
                        v[j] = *reinterpret_cast<const float4*>(row + (j * 32 + lane) * 4);
                        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
                    }
                const float mean = warp_sum(s) / (float)K;
                float q = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < nv) {
                        const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                        q += (a * a + b * b) + (c * c + d * d);
                    }
                const float inv = 1.f / sqrtf(warp_sum(q) / (float)K + eps);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < nv) {
                        const int i = (j * 32 + lane) * 4;
                        const float4 gm = *reinterpret_cast<const float4*>(gamma + i);
                        const float4 bt = *reinterpret_cast<const float4*>(beta + i);
                        __nv_bfloat162 lo = __floats2bfloat162_rn((v[j].x - mean) * inv * gm.x + bt.x,
                                                                  (v[j].y - mean) * inv * gm.y + bt.y);
                        __nv_bfloat162 hi = __floats2bfloat162_rn((v[j].z - mean) * inv * gm.z + bt.z,
                                                                  (v[j].w - mean) * inv * gm.w + bt.w);
                        *reinterpret_cast<__nv_bfloat162*>(dst + i) = lo;
                        *reinterpret_cast<__nv_bfloat162*>(dst + i + 2) = hi;
                    }
                continue;
            }
            float s = 0.f;
            for (int i = lane; i < K; i += 32) s += row[i];
            const float mean = warp_sum(s) / (float)K;
            float q = 0.f;
            for (int i = lane; i < K; i += 32) { const float c = row[i] - mean; q += c * c; }
            const float inv = 1.f / sqrtf(warp_sum(q) / (float)K + eps);
            for (int i = lane; i < K; i += 32)
                dst[i] = __float2bfloat16_rn((row[i] - mean) * inv * gamma[i] + beta[i]);
        }
        __syncthreads();
    }

    float acc[MT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    if (n0 < N) {
        const __nv_bfloat16* w_lo = W + (size_t)min(n0 + g, N - 1) * K + t * 8;
        const __nv_bfloat16* w_hi = W + (size_t)min(n0 + g + 8, N - 1) * K + t * 8;
        const __nv_bfloat16* Xb = reinterpret_cast<const __nv_bfloat16*>(Xv);
        const int n_chunks = K / 32;
        // chunk c belongs to k-part (c % ksplit); this warp walks c = kpart, kpart + ksplit, …
        for (int c0 = kpart; c0 < n_chunks; c0 += ksplit * UNROLL) {
            uint4 wl[UNROLL], wh[UNROLL];
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int c = c0 + u * ksplit;
                if (c < n_chunks) {
                    wl[u] = ldg16_stream(w_lo + c * 32);
                    wh[u] = ldg16_stream(w_hi + c * 32);
                }
            }
#pragma unroll
            for (int u = 0; u < UNROLL; ++u) {
                const int c = c0 + u * ksplit;
                if (c < n_chunks) {
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        uint4 x;
                        if (LN) {
                            x = *reinterpret_cast<const uint4*>(xs + (size_t)(mt * 8 + g) * xs_stride + (c * 32 + t * 8) * 2);
                        } else {
                            x = ldg16(Xb + (size_t)min(mt * 8 + g, M - 1) * ldx + c * 32 + t * 8);
                        }
                        mma_bf16(acc[mt], wl[u].x, wh[u].x, wl[u].y, wh[u].y, x.x, x.y);
                        mma_bf16(acc[mt], wl[u].z, wh[u].z, wl[u].w, wh[u].w, x.z, x.w);
                    }
                }
            }
        }
    }

    // partial sums of the k-parts: added in the order of the parts by the first warp of each group
    if (ksplit > 1) {
        float* mine = red + (size_t)warp * (MT * 4 * 32);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int j = 0; j < 4; ++j) mine[(mt * 4 + j) * 32 + lane] = acc[mt][j];
        __syncthreads();
        if (kpart != 0) return;
        for (int p = 1; p < ksplit; ++p) {
            const float* other = red + (size_t)(warp + p) * (MT * 4 * 32);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[mt][j] += other[(mt * 4 + j) * 32 + lane];
        }
    }
    if (n0 >= N) return;

    // epilogue: thread holds columns n0+g and n0+g+8 for rows mt*8 + 2t, 2t+1
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + g + ((j & 2) ? 8 : 0);
            const int m = mt * 8 + 2 * t + (j & 1);
            if (n >= N || m >= M) continue;
            float v = acc[mt][j];
            if (bias) v += bias[n];
            v = apply_act_rt(v, act);
            if (residual) v += residual[(size_t)m * ldy + n];
            ElemIO<OT>::store(Y + (size_t)m * ldy + n, v);
            if (kv.Kc != nullptr && n >= kv.k_off) {
                const bool is_v = n >= kv.v_off;
                const int col = n - (is_v ? kv.v_off : kv.k_off);
                if (col < kv.width) {
                    const int slot = kv.tok_slot[m];
                    if (slot >= 0) {
                        const int pos = kv.tok_pos[m];
                        const int blk = kv.block_table[(size_t)slot * kv.max_blocks + pos / kv.BT];
                        if (blk >= 0) {
                            const int h = col / kv.dh, cc = col - h * kv.dh;
                            const size_t dst = (((size_t)blk * kv.Hkv + h) * kv.BT + (pos % kv.BT)) * kv.dh + cc;
                            __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(is_v ? kv.Vc : kv.Kc);
                            base[dst] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
        }
    }
}

template <int MT, bool LN, typename OT>
int launch(const void* X, const void* W, const float* bias, const float* residual, void* Y, int M, int N, int K,
           int ldx, int ldy, int act, int ksplit, const float* gamma, const float* beta, float eps,
           const KvScatter& kv, cudaStream_t stream) {
    const int groups_per_cta = SK_WARPS / ksplit;
    const int n_groups = (N + 15) / 16;
    const int grid = (n_groups + groups_per_cta - 1) / groups_per_cta;
    const int xs_stride = LN ? (K * 2 + 64 + ((128 - (K * 2) % 128) % 128)) : 0;
    const size_t smem = (size_t)xs_stride * MT * 8 + (ksplit > 1 ? (size_t)SK_WARPS * MT * 4 * 32 * sizeof(float) : 0);
    auto kern = gemm_skinny_kernel<MT, LN, OT>;
    static size_t allowed = 48 * 1024;   // per instantiation: the attribute is raised once, not per launch
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_skinny: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        allowed = smem;
    }
    kern<<<grid, SK_THREADS, smem, stream>>>(X, (const __nv_bfloat16*)W, bias, residual, (OT*)Y, M, N, K, ldx, ldy,
                                              act, ksplit, gamma, beta, eps, kv);
    return vlrf_check_launch("gemm_skinny");
}

template <bool LN, typename OT>
int dispatch_mt(int mt, const void* X, const void* W, const float* bias, const float* residual, void* Y, int M,
                int N, int K, int ldx, int ldy, int act, int ksplit, const float* gamma, const float* beta,
                float eps, const KvScatter& kv, cudaStream_t stream) {
    switch (mt) {
        case 1: return launch<1, LN, OT>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
        case 2: return launch<2, LN, OT>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
        case 4: return launch<4, LN, OT>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
        default: return launch<8, LN, OT>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
    }
}
}  // namespace

// The largest width for which the LayerNorm-fused form holds its normalised rows in shared memory.
extern "C" int vlrf_gemm_skinny_ln_fits(int M, int K) {
    const int mt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
    const int xs_stride = K * 2 + 64 + ((128 - (K * 2) % 128) % 128);
    const size_t smem = (size_t)xs_stride * mt * 8 + (size_t)SK_WARPS * mt * 4 * 32 * sizeof(float);
    return smem <= 200 * 1024 ? 1 : 0;
}

extern "C" int vlrf_gemm_skinny(const void* X, int x_is_f32_ln, const void* W, const float* bias,
                                const float* residual, void* Y, int out_dtype, int M, int N, int K, int ldx,
                                int ldy, int act, const float* gamma, const float* beta, float eps,
                                // optional scatter of K/V columns into the cache (Kc == nullptr: none)
                                void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                                const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT,
                                int sm_count, cudaStream_t stream) {
    VLRF_REQUIRE(M >= 1 && M <= 64, "gemm_skinny: takes 1…64 rows, not %d", M);
    VLRF_REQUIRE(N > 0 && K > 0 && K % 32 == 0, "gemm_skinny: K=%d must be a positive multiple of 32", K);
    VLRF_REQUIRE(ldx >= K && ldy >= N, "gemm_skinny: leading sizes too small");
    VLRF_REQUIRE(ldx % 8 == 0 || x_is_f32_ln, "gemm_skinny: bf16 rows must start on 16-byte boundaries (ldx=%d)", ldx);
    VLRF_REQUIRE(act >= 0 && act <= 2, "gemm_skinny: unknown activation %d", act);
    VLRF_REQUIRE(!x_is_f32_ln || (gamma && beta), "gemm_skinny: the fused LayerNorm needs weight and bias");
    VLRF_REQUIRE(!x_is_f32_ln || vlrf_gemm_skinny_ln_fits(M, K), "gemm_skinny: %d rows of width %d do not fit the fused LayerNorm", M, K);
    KvScatter kv{};
    if (Kc != nullptr) {
        VLRF_REQUIRE(Vc && block_table && tok_slot && tok_pos && Hkv > 0 && dh > 0 && BT > 0 && max_blocks > 0,
                     "gemm_skinny: incomplete cache scatter arguments");
        VLRF_REQUIRE(out_dtype == VLRF_BF16, "gemm_skinny: the cache scatter writes bfloat16");
        kv = KvScatter{Kc, Vc, block_table, tok_slot, tok_pos, max_blocks, k_off, v_off, Hkv * dh, dh, Hkv, BT};
    }
    const int mt = M <= 8 ? 1 : M <= 16 ? 2 : M <= 32 ? 4 : 8;
    // as many warps per 16 columns as it takes to give every SM work, within what K allows
    const int n_groups = (N + 15) / 16;
    int ksplit = 1;
    while (ksplit < SK_WARPS && (n_groups * ksplit + SK_WARPS - 1) / SK_WARPS < sm_count && K / 32 >= ksplit * 2) ksplit *= 2;
    if (x_is_f32_ln) {
        if (out_dtype == VLRF_BF16)
            return dispatch_mt<true, __nv_bfloat16>(mt, X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
        if (out_dtype == VLRF_F32)
            return dispatch_mt<true, float>(mt, X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
    } else {
        if (out_dtype == VLRF_BF16)
            return dispatch_mt<false, __nv_bfloat16>(mt, X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
        if (out_dtype == VLRF_F32)
            return dispatch_mt<false, float>(mt, X, W, bias, residual, Y, M, N, K, ldx, ldy, act, ksplit, gamma, beta, eps, kv, stream);
    }
    return vlrf_fail(VLRF_ERR_INVALID_ARG, "gemm_skinny: unknown output dtype %d", out_dtype);
}
