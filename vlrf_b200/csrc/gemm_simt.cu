// Y[M,N] = act(X[M,K] · W[N,K]^T + bias[N]) (+ residual[M,N]) on the CUDA cores with float32 FMAs.
//
// This is the matrix product of the true 32-bit path (no tensor-core mode of reduced precision
// is involved) and the fallback of the bfloat16 path for shapes that the tensor-core kernels
// refuse.  W is kept [out, in] with `in` contiguous, so the product is the reference's
// linear(x, W) = x · Wᵀ (include/model/compute.hpp:64-68) with bias (include/model/attention.hpp:103-105),
// activation (include/model/feedforward.hpp:54-76) and residual (include/model/transformer_block.hpp:153,158)
// applied in the epilogue.  Each output element accumulates over K in the same order whatever M
// is, so a row's result does not depend on how many rows share the call.
#include "common.cuh"

namespace {
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4, THREADS = 256;

template <typename IT, typename OT>
__global__ void __launch_bounds__(THREADS)
gemm_simt_kernel(const IT* __restrict__ X, const IT* __restrict__ W, const float* __restrict__ bias,
                 const float* residual, OT* Y, int M, int N, int K, int ldx, int ldy, int act) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int lr = tid >> 2;         // 0..63: row of the tile this thread loads
    const int lk = (tid & 3) * 4;    // 0,4,8,12: first of its 4 k's
    const int ty = tid >> 4, tx = tid & 15;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int k = k0 + lk + j;
            const int gm = m0 + lr, gn = n0 + lr;
            As[lk + j][lr] = (gm < M && k < K) ? ElemIO<IT>::load(X + (size_t)gm * ldx + k) : 0.f;
            Bs[lk + j][lr] = (gn < N && k < K) ? ElemIO<IT>::load(W + (size_t)gn * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = Bs[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (bias) v += bias[n];
            v = apply_act_rt(v, act);
            if (residual) v += residual[(size_t)m * ldy + n];
            ElemIO<OT>::store(Y + (size_t)m * ldy + n, v);
        }
    }
}
}  // namespace

extern "C" int vlrf_gemm_simt(const void* X, const void* W, const float* bias, const float* residual,
                              void* Y, int M, int N, int K, int ldx, int ldy, int in_dtype, int out_dtype,
                              int act, cudaStream_t stream) {
    VLRF_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    VLRF_REQUIRE(ldx >= K && ldy >= N, "gemm: leading sizes ldx=%d ldy=%d are smaller than K=%d N=%d", ldx, ldy, K, N);
    VLRF_REQUIRE(act >= 0 && act <= 2, "gemm: unknown activation %d", act);
    if (M == 0) return VLRF_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    VLRF_REQUIRE(grid.y <= 65535, "gemm: M=%d needs more than 65535 row tiles", M);
#define LAUNCH(IT, OT)                                                                                  \
    gemm_simt_kernel<IT, OT><<<grid, THREADS, 0, stream>>>((const IT*)X, (const IT*)W, bias, residual, \
                                                           (OT*)Y, M, N, K, ldx, ldy, act)
    if (in_dtype == VLRF_F32 && out_dtype == VLRF_F32) LAUNCH(float, float);
    else if (in_dtype == VLRF_BF16 && out_dtype == VLRF_F32) LAUNCH(__nv_bfloat16, float);
    else if (in_dtype == VLRF_BF16 && out_dtype == VLRF_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else return vlrf_fail(VLRF_ERR_INVALID_ARG, "gemm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
    return vlrf_check_launch("gemm_simt");
}
