// Y[M,N] = act(X[M,K] · W[N,K]^T + bias) (+ residual) on the 5th-generation tensor cores (tcgen05), for
// the many-row products of a prompt step.  bfloat16 operands, float32 accumulation in tensor memory.
//
// One CTA computes a 128 × BN tile of Y.  Its six warps have fixed jobs:
//   warp 4  producer: for every 64-wide k block it waits until the ring stage is free, announces the
//           bytes on the stage's "full" mbarrier and issues two tiled TMA loads (128 rows of X, BN rows of
//           W; 128-byte swizzle; rows and columns outside the matrices read as zeros);
//   warp 5  one elected thread issues the MMAs: four `tcgen05.mma.cta_group::1.kind::f16` of shape
//           128 × BN × 16 per k block, operands straight from shared memory through matrix descriptors,
//           accumulator in tensor memory; `tcgen05.commit` frees the stage when those MMAs have read it,
//           and after the last k block signals the accumulator as complete;
//   warps 0-3  epilogue: each reads its 32 lanes of the accumulator with `tcgen05.ld`, adds bias, applies
//           GELU, adds the float32 residual (reference: include/model/feedforward.hpp:54-76,
//           include/model/transformer_block.hpp:153,158) and stores bfloat16 or float32 rows.
// Tensor memory (BN columns) is allocated by warp 4 and freed by it at the end on every path.  Every
// mbarrier wait is bounded; a wait that gives up sets a bit in the device error word, and the CTA still
// frees its tensor memory and returns.
//
// The product is the reference's linear(x, W) = x · Wᵀ (include/model/compute.hpp:64-68).
#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;
constexpr int TC_THREADS = 192;
constexpr uint32_t TC_WAIT_LIMIT = 1u << 21;

// Optional scatter of the K and V columns of a fused q/k/v projection into one layer's paged cache
// (reference: include/model/kv_cache.hpp:215-251).  Kc == nullptr: none.
struct TcKvScatter {
    void* Kc; void* Vc;            // [block][kv_head][BT][dh], bf16
    const int* block_table; const int* tok_slot; const int* tok_pos;
    int max_blocks, k_off, v_off, width, dh, Hkv, BT;   // width = Hkv*dh
};

__device__ __forceinline__ uint32_t tsm(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void tbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(tsm(bar)), "r"(count));
}
__device__ __forceinline__ void tbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(tsm(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool tbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(tsm(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// false if the wait gave up
__device__ __forceinline__ bool tbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_WAIT_LIMIT; ++i)
        if (tbar_try_wait(bar, parity)) return true;
    return false;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes (64 bf16) written by TMA with
// the 128-byte swizzle: 8-row groups are 1024 bytes apart; version 1 (Blackwell); layout type 2 (128B swizzle).
__device__ __forceinline__ uint64_t umma_desc_k128(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((tsm(tile) >> 4) & 0x3FFF);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused with swizzle): 1
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows × 128 bytes
    d |= (uint64_t)1 << 46;                               // descriptor version
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D float32, A and B bfloat16, both K-major, shape M × N
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tsm(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

// SWAP: the roles of the two matrices are exchanged — the 128-row operand is W (tmap_x then describes W),
// the BN-row operand is X with its few rows — so that a product with few rows still fills the 128-row MMA.
// The accumulator then holds Yᵀ: lane = output column n, TMEM column = row m; the epilogue writes Y[m][n],
// for each m 32 consecutive n per warp.
template <int BN, int STAGES, typename OT, bool SWAP>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const float* __restrict__ bias, const float* residual, OT* Y, int M, int N, int K, int ldy,
                    int act, TcKvScatter kv, int* __restrict__ dev_err) {
    extern __shared__ unsigned char tc_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int A_BYTES = TC_BM * TC_BK * 2, B_BYTES = BN * TC_BK * 2;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;       // tensor memory is allocated in powers of two from 32 columns
    unsigned char* a_tiles = smem;                                   // [STAGES][128][128 B]
    unsigned char* b_tiles = smem + (size_t)STAGES * A_BYTES;        // [STAGES][BN][128 B]
    uint64_t* full = reinterpret_cast<uint64_t*>(b_tiles + (size_t)STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_done = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_done + 1);
    int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // not swapped: m0 = first row of X, n0 = first row of W.  Swapped: m0 = first row of W (output column), n0 = 0.
    const int m0 = SWAP ? blockIdx.x * TC_BM : blockIdx.y * TC_BM, n0 = SWAP ? 0 : blockIdx.x * BN;
    const int n_kb = (K + TC_BK - 1) / TC_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { tbar_init(&full[s], 1); tbar_init(&empty[s], 1); }
        tbar_init(acc_done, 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        if (lane == 0) { tma_prefetch_descriptor(&tmap_x); tma_prefetch_descriptor(&tmap_w); }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tsm(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    pdl_launch_dependents();
    pdl_wait();                                    // X (and the residual) come from the kernel before

    if (warp == 4) {
        if (lane == 0) {
            for (int kb = 0; kb < n_kb; ++kb) {
                const int s = kb % STAGES;
                if (kb >= STAGES && !tbar_wait(&empty[s], ((kb / STAGES) - 1) & 1)) { atomicExch(s_abort, 1); break; }
                tbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                tma_load_2d(a_tiles + (size_t)s * A_BYTES, &tmap_x, kb * TC_BK, m0, &full[s]);
                tma_load_2d(b_tiles + (size_t)s * B_BYTES, &tmap_w, kb * TC_BK, n0, &full[s]);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
            bool ok = true;
            for (int kb = 0; kb < n_kb && ok; ++kb) {
                const int s = kb % STAGES;
                if (!tbar_wait(&full[s], (kb / STAGES) & 1)) { atomicExch(s_abort, 1); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc_k128(a_tiles + (size_t)s * A_BYTES);
                const uint64_t db = umma_desc_k128(b_tiles + (size_t)s * B_BYTES);
#pragma unroll
                for (int k = 0; k < TC_BK / 16; ++k)          // 16 elements = 32 bytes = 2 descriptor units along K
                    umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);                       // the stage is free once these MMAs have read it
            }
            umma_commit(acc_done);                            // arrives when every MMA issued so far is complete
        }
    } else {
        // epilogue: warp w reads accumulator lanes 32w … 32w+31 = rows m0 + 32w + lane
        const bool have = tbar_wait(acc_done, 0);
        if (!have) atomicExch(s_abort, 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int m = m0 + warp * 32 + lane;
        // where this thread's row goes in the cache, if the product feeds one
        int kv_blk = -2, kv_row = 0;                   // −2: nothing to write
        if (kv.Kc != nullptr && m < M) {
            const int slot = kv.tok_slot[m];
            if (slot >= 0) {
                const int pos = kv.tok_pos[m];
                kv_blk = kv.block_table[(size_t)slot * kv.max_blocks + pos / kv.BT];
                kv_row = pos % kv.BT;
                if (kv_blk < 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
            }
        }
        if (SWAP) {
            if (have && !*s_abort) {
                const int n = m0 + warp * 32 + lane;          // this thread's output column = row of W
                const float bv = (bias && n < N) ? bias[n] : 0.f;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t r[16];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                        : "r"(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0));
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (n < N) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int m = c0 + j;
                            if (m < M) {
                                float x = apply_act_rt(__uint_as_float(r[j]) + bv, act);
                                if (residual) x += residual[(size_t)m * ldy + n];
                                ElemIO<OT>::store(Y + (size_t)m * ldy + n, x);
                            }
                        }
                    }
                }
            }
        } else if (have && !*s_abort) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (m < M && n0 + c0 < N) {
                    const int n_here = min(32, N - (n0 + c0));
                    OT* yrow = Y + (size_t)m * ldy + n0 + c0;
                    const float* rrow = residual ? residual + (size_t)m * ldy + n0 + c0 : nullptr;
                    const float* brow = bias ? bias + n0 + c0 : nullptr;
                    if (n_here == 32 && (ldy % 8) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) {
                                float x = __uint_as_float(r[j + e]);
                                if (brow) x += __ldg(brow + j + e);
                                v[e] = apply_act_rt(x, act);
                            }
                            if (rrow) {
                                const float4 r0 = *reinterpret_cast<const float4*>(rrow + j);
                                const float4 r1 = *reinterpret_cast<const float4*>(rrow + j + 4);
                                v[0] += r0.x; v[1] += r0.y; v[2] += r0.z; v[3] += r0.w;
                                v[4] += r1.x; v[5] += r1.y; v[6] += r1.z; v[7] += r1.w;
                            }
                            if (sizeof(OT) == 4) {
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(yrow) + j) = make_float4(v[0], v[1], v[2], v[3]);
                                *reinterpret_cast<float4*>(reinterpret_cast<float*>(yrow) + j + 4) = make_float4(v[4], v[5], v[6], v[7]);
                            } else {
                                uint4 pk;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[4], v[5]), p3 = __floats2bfloat162_rn(v[6], v[7]);
                                pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
                                pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
                                *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(yrow) + j) = pk;
                                const int n = n0 + c0 + j;                 // 8 columns: one head, one of q / k / v
                                if (kv_blk >= 0 && n >= kv.k_off) {
                                    const bool is_v = n >= kv.v_off;
                                    const int col = n - (is_v ? kv.v_off : kv.k_off);
                                    if (col < kv.width) {
                                        const int hh = col / kv.dh, cc = col - hh * kv.dh;
                                        __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(is_v ? kv.Vc : kv.Kc);
                                        *reinterpret_cast<uint4*>(base + (((size_t)kv_blk * kv.Hkv + hh) * kv.BT + kv_row) * kv.dh + cc) = pk;
                                    }
                                }
                            }
                        }
                    } else {
                        for (int j = 0; j < n_here; ++j) {
                            float x = __uint_as_float(r[j]);
                            if (brow) x += brow[j];
                            x = apply_act_rt(x, act);
                            if (rrow) x += rrow[j];
                            ElemIO<OT>::store(yrow + j, x);
                            const int n = n0 + c0 + j;
                            if (kv_blk >= 0 && n >= kv.k_off) {
                                const bool is_v = n >= kv.v_off;
                                const int col = n - (is_v ? kv.v_off : kv.k_off);
                                if (col < kv.width) {
                                    const int hh = col / kv.dh, cc = col - hh * kv.dh;
                                    __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(is_v ? kv.Vc : kv.Kc);
                                    base[(((size_t)kv_blk * kv.Hkv + hh) * kv.BT + kv_row) * kv.dh + cc] = __float2bfloat16_rn(x);
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    // everyone meets here on every path; then the allocating warp gives the tensor memory back
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *s_abort) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
}

template <int BN, int STAGES, typename OT, bool SWAP = false>
int launch_tc(const void* X, const void* W, const float* bias, const float* residual, void* Y, int M, int N, int K,
              int ldx, int ldy, int act, const TcKvScatter& kv, int* dev_err, cudaStream_t stream) {
    CUtensorMap tx, tw;      // tx: the 128-row operand, tw: the BN-row operand
    int st = SWAP ? vlrf_make_tmap_bf16(W, N, K, K, TC_BM, TC_BK, &tx) : vlrf_make_tmap_bf16(X, M, K, ldx, TC_BM, TC_BK, &tx);
    if (st != VLRF_OK) return st;
    st = SWAP ? vlrf_make_tmap_bf16(X, M, K, ldx, BN, TC_BK, &tw) : vlrf_make_tmap_bf16(W, N, K, K, BN, TC_BK, &tw);
    if (st != VLRF_OK) return st;
    const size_t smem = 1024 + (size_t)STAGES * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 1) * 8 + 16;
    auto kern = gemm_tcgen05_kernel<BN, STAGES, OT, SWAP>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_tcgen05: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + TC_BM - 1) / TC_BM);
    if (SWAP) grid = dim3((N + TC_BM - 1) / TC_BM, 1);
    cudaError_t e = launch_chained(kern, grid, dim3(TC_THREADS), smem, stream, tx, tw, bias, residual, (OT*)Y, M, N, K, ldy,
                                   act, kv, dev_err);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_tcgen05: %s", cudaGetErrorString(e));
    return vlrf_check_launch("gemm_tcgen05");
}
}  // namespace

// Whether this kernel takes the shape (bfloat16 only): rows must start on 16-byte boundaries for TMA.
extern "C" int vlrf_gemm_tcgen05_takes(int M, int N, int K, int ldx) {
    return (M >= 1 && N >= 1 && K >= 8 && K % 8 == 0 && ldx % 8 == 0) ? 1 : 0;
}

extern "C" int vlrf_gemm_tcgen05(const void* X, const void* W, const float* bias, const float* residual, void* Y,
                                 int M, int N, int K, int ldx, int ldy, int out_dtype, int act,
                                 // optional scatter of K/V columns into the cache (Kc == nullptr: none)
                                 void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                                 const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT, int* dev_err,
                                 cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_gemm_tcgen05_takes(M, N, K, ldx), "gemm_tcgen05: M=%d N=%d K=%d ldx=%d: K and the row stride must be multiples of 8", M, N, K, ldx);
    VLRF_REQUIRE(ldy >= N && act >= 0 && act <= 2 && dev_err != nullptr, "gemm_tcgen05: bad arguments");
    VLRF_REQUIRE((M + TC_BM - 1) / TC_BM <= 65535, "gemm_tcgen05: too many row tiles");
    TcKvScatter kv{};
    if (Kc != nullptr) {
        VLRF_REQUIRE(Vc && block_table && tok_slot && tok_pos && Hkv > 0 && dh > 0 && BT > 0 && max_blocks > 0,
                     "gemm_tcgen05: incomplete cache scatter arguments");
        VLRF_REQUIRE(out_dtype == VLRF_BF16 && dh % 8 == 0 && k_off % 8 == 0 && v_off % 8 == 0,
                     "gemm_tcgen05: the cache scatter writes bfloat16 heads of a multiple of 8 columns");
        kv = TcKvScatter{Kc, Vc, block_table, tok_slot, tok_pos, max_blocks, k_off, v_off, Hkv * dh, dh, Hkv, BT};
    }
    if (M <= 64 && Kc == nullptr) {
        // few rows: W fills the 128-row operand, the rows of X are the MMA's N
#define SWAPPED(BNV) (out_dtype == VLRF_BF16 ? launch_tc<BNV, 4, __nv_bfloat16, true>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream) \
                                             : launch_tc<BNV, 4, float, true>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream))
        VLRF_REQUIRE(out_dtype == VLRF_BF16 || out_dtype == VLRF_F32, "gemm_tcgen05: unknown output dtype %d", out_dtype);
        if (M <= 16) return SWAPPED(16);
        if (M <= 32) return SWAPPED(32);
        return SWAPPED(64);
#undef SWAPPED
    }
    // narrower tiles when wide ones would leave most SMs idle
    const long long tiles128 = (long long)((N + 127) / 128) * ((M + 127) / 128);
    const bool narrow = tiles128 < 120;
    if (out_dtype == VLRF_BF16) {
        if (narrow) return launch_tc<64, 4, __nv_bfloat16>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream);
        return launch_tc<128, 3, __nv_bfloat16>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream);
    }
    if (out_dtype == VLRF_F32) {
        if (narrow) return launch_tc<64, 4, float>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream);
        return launch_tc<128, 3, float>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream);
    }
    return vlrf_fail(VLRF_ERR_INVALID_ARG, "gemm_tcgen05: unknown output dtype %d", out_dtype);
}
