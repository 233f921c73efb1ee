// Y[M,N] = act(X[M,K] · W[N,K]^T + bias) (+ residual) on the 5th-generation tensor cores (tcgen05), for
// the many-row products of a prompt step.  bfloat16 operands, float32 accumulation in tensor memory.
//
// A persistent CTA computes 128 × BN tiles of Y, one after another.  Its ten warps have fixed jobs:
//   warp 8  producer: for every 64-wide k block it waits until the ring stage is free, announces the
//           bytes on the stage's "full" mbarrier and issues two tiled TMA loads (128 rows of X, BN rows of
//           W; 128-byte swizzle; rows and columns outside the matrices read as zeros);
//   warp 9  one elected thread issues the MMAs: four `tcgen05.mma.cta_group::1.kind::f16` of shape
//           128 × BN × 16 per k block, operands straight from shared memory through matrix descriptors,
//           accumulator in tensor memory (two accumulators alternate, so a tile's epilogue overlaps the
//           next tile's MMAs); `tcgen05.commit` frees the stage when those MMAs have read it, and after the
//           last k block signals the accumulator as complete;
//   warps 0-7  epilogue: two warps share 32 lanes of the accumulator and take half of its columns each;
//           they read them with `tcgen05.ld` (bias and residual are fetched while that is in flight), add bias, apply
//           GELU, adds the float32 residual (reference: include/model/feedforward.hpp:54-76,
//           include/model/transformer_block.hpp:153,158) and stores bfloat16 or float32 rows.
// Tensor memory (2·BN columns) is allocated by warp 8 and freed by it at the end on every path.  Every
// mbarrier wait is bounded; a wait that gives up sets a bit in the device error word, and the CTA still
// frees its tensor memory and returns.
//
// The product is the reference's linear(x, W) = x · Wᵀ (include/model/compute.hpp:64-68).
#include <type_traits>
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

namespace {

int sm_count_cached() {                          // asked once: the query is slow next to a launch
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        sms = v > 0 ? v : 148;
    }
    return sms;
}

constexpr int TC_BM = 128;
constexpr int TC_BK = 64;           // elements of K in one 128-byte swizzle atom: what one TMA load and one descriptor cover
// Atoms of K in a stage of the ring.  One thread issues the MMAs, and a stage costs it about 550 cycles whatever
// the tile's width: some 63 for each of an atom's four MMAs, the rest for the wait, the commit and the loop.  The
// tensor pipe needs 4 x 186 cycles for an atom of a 256-wide tile but only 4 x 70 of a 96-wide one, so narrow
// tiles take two atoms a stage and pay the fixed part half as often.
__host__ __device__ constexpr int tc_atoms(int bn) { return bn <= 128 ? 2 : 1; }
constexpr int TC_THREADS = 320;      // warps 0-7: epilogue (two per 32 accumulator lanes), 8: producer, 9: MMA issue

// Optional scatter of the K and V columns of a fused q/k/v projection into one layer's paged cache
// (reference: include/model/kv_cache.hpp:215-251).  Kc == nullptr: none.
struct TcKvScatter {
    void* Kc; void* Vc;            // [block][kv_head][BT][dh], bf16
    const int* block_table; const int* tok_slot; const int* tok_pos;
    int max_blocks, k_off, v_off, width, dh, Hkv, BT;   // width = Hkv*dh
};

// SWAP: the roles of the two matrices are exchanged — the 128-row operand is W (tmap_x then describes W),
// the BN-row operand is X with its few rows — so that a product with few rows still fills the 128-row MMA.
// The accumulator then holds Yᵀ: lane = output column n, TMEM column = row m; the epilogue writes Y[m][n],
// for each m 32 consecutive n per warp.
//
// The CTA is persistent: it takes the output tiles blockIdx.x, + gridDim.x, …  Tensor memory holds two
// accumulators, so the epilogue of one tile runs while the MMAs of the next fill the other, and the
// producer keeps the shared-memory ring full across tile boundaries.
template <int BN, int STAGES, typename OT, bool SWAP>
__global__ void __launch_bounds__(TC_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                    const float* __restrict__ bias, const float* residual, OT* Y, int M, int N, int K, int ldy,
                    int act, TcKvScatter kv, int* __restrict__ dev_err, long long* trace) {
    extern __shared__ unsigned char tc_raw[];
    // (stations of the time stamps, kind 3: 0 the CTA begins, 1 the kernel ahead has finished, 2 the first tile's
    // accumulator is complete, 3 the last tile's, 6 the last tile is stored; thread 0 stamps)
    if (threadIdx.x == 0) VLRF_TRACE(trace, 3, (int)blockIdx.x, 0);
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int KA = tc_atoms(BN);
    constexpr int A_ATOM = TC_BM * TC_BK * 2, B_ATOM = BN * TC_BK * 2;           // bytes of one atom of each operand
    constexpr int A_BYTES = KA * A_ATOM, B_BYTES = KA * B_ATOM;
    // two accumulators, ACC_STRIDE columns apart; the allocation is a power of two ≥ 32
    constexpr int ACC_STRIDE = BN <= 16 ? 16 : (BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256)));
    constexpr int TMEM_COLS = 2 * ACC_STRIDE < 32 ? 32 : 2 * ACC_STRIDE;
    unsigned char* a_tiles = smem;                                   // [STAGES][KA][128][128 B]
    unsigned char* b_tiles = smem + (size_t)STAGES * A_BYTES;        // [STAGES][KA][BN][128 B]
    uint64_t* full = reinterpret_cast<uint64_t*>(b_tiles + (size_t)STAGES * B_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;                             // [2] MMAs of a tile are complete
    uint64_t* acc_empty = acc_full + 2;                              // [2] the epilogue has read the accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_kb = (K + KA * TC_BK - 1) / (KA * TC_BK);             // stages of K (atoms behind K's end are read as zeros)
    // tiles: not swapped — 128 rows of X by BN rows of W, neighbours in N first (they share the rows of X in
    // L2); swapped — 128 rows of W by all rows of X
    const int tiles_n = SWAP ? 1 : (N + BN - 1) / BN;
    const int n_tiles = SWAP ? (N + TC_BM - 1) / TC_BM : tiles_n * ((M + TC_BM - 1) / TC_BM);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { tbar_init(&full[s], 1); tbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { tbar_init(&acc_full[b], 1); tbar_init(&acc_empty[b], 8); }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        if (lane == 0) { tma_prefetch_descriptor(&tmap_x); tma_prefetch_descriptor(&tmap_w); }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tsm(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // The weights do not depend on the kernel ahead: the first tile's weight operand (the 128-row one when the
    // roles are exchanged, else the BN-row one) is requested for as many k blocks as the ring holds before the
    // wait; the rows of X follow after it.
    const int early = (int)blockIdx.x < n_tiles ? min(STAGES, n_kb) : 0;
    if (warp == 8 && lane == 0) {
        const int tile = blockIdx.x;
        const int m0 = SWAP ? tile * TC_BM : (tile / tiles_n) * TC_BM, n0 = SWAP ? 0 : (tile % tiles_n) * BN;
        for (int kb = 0; kb < early; ++kb) {
            tbar_expect_tx(&full[kb], A_BYTES + B_BYTES);
#pragma unroll
            for (int a = 0; a < KA; ++a) {
                if (SWAP) tma_load_2d(a_tiles + (size_t)kb * A_BYTES + a * A_ATOM, &tmap_x, (kb * KA + a) * TC_BK, m0, &full[kb]);
                else tma_load_2d(b_tiles + (size_t)kb * B_BYTES + a * B_ATOM, &tmap_w, (kb * KA + a) * TC_BK, n0, &full[kb]);
            }
        }
    }
    pdl_launch_dependents();
    pdl_wait();                                    // X (and the residual) come from the kernel before
    if (threadIdx.x == 0) VLRF_TRACE(trace, 3, (int)blockIdx.x, 1);

    if (warp == 8) {
        if (lane == 0) {
            uint32_t kc = 0;                       // k-blocks requested so far, over all tiles
            for (int tile = blockIdx.x; tile < n_tiles && !*(volatile int*)s_abort; tile += gridDim.x) {
                const int m0 = SWAP ? tile * TC_BM : (tile / tiles_n) * TC_BM, n0 = SWAP ? 0 : (tile % tiles_n) * BN;
                for (int kb = 0; kb < n_kb; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    const uint32_t use = kc / STAGES;
                    if ((int)kc < early) {         // the weight half of this stage is already on its way
#pragma unroll
                        for (int a = 0; a < KA; ++a) {
                            if (SWAP) tma_load_2d(b_tiles + (size_t)s * B_BYTES + a * B_ATOM, &tmap_w, (kb * KA + a) * TC_BK, n0, &full[s]);
                            else tma_load_2d(a_tiles + (size_t)s * A_BYTES + a * A_ATOM, &tmap_x, (kb * KA + a) * TC_BK, m0, &full[s]);
                        }
                        continue;
                    }
                    if (use >= 1 && !tbar_wait_or_abort(&empty[s], (use - 1) & 1, s_abort)) { atomicExch(s_abort, 1); break; }
                    tbar_expect_tx(&full[s], A_BYTES + B_BYTES);
#pragma unroll
                    for (int a = 0; a < KA; ++a) {
                        tma_load_2d(a_tiles + (size_t)s * A_BYTES + a * A_ATOM, &tmap_x, (kb * KA + a) * TC_BK, m0, &full[s]);
                        tma_load_2d(b_tiles + (size_t)s * B_BYTES + a * B_ATOM, &tmap_w, (kb * KA + a) * TC_BK, n0, &full[s]);
                    }
                }
            }
        }
    } else if (warp == 9) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, BN);
            uint32_t kc = 0, tc = 0;
            for (int tile = blockIdx.x; tile < n_tiles && !*(volatile int*)s_abort; tile += gridDim.x, ++tc) {
                const uint32_t b = tc & 1, use = tc >> 1;
                if (use >= 1 && !tbar_wait_or_abort(&acc_empty[b], (use - 1) & 1, s_abort)) { atomicExch(s_abort, 1); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t tmem_d = tmem_base + b * ACC_STRIDE;
                bool ok = true;
                for (int kb = 0; kb < n_kb; ++kb, ++kc) {
                    const int s = kc % STAGES;
                    if (!tbar_wait_or_abort(&full[s], (kc / STAGES) & 1, s_abort)) { atomicExch(s_abort, 1); ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t da = umma_desc_k128(a_tiles + (size_t)s * A_BYTES);
                    const uint64_t db = umma_desc_k128(b_tiles + (size_t)s * B_BYTES);
#pragma unroll
                    for (int a = 0; a < KA; ++a) {
#pragma unroll
                        for (int k = 0; k < TC_BK / 16; ++k)  // 16 elements = 32 bytes = 2 descriptor units along K
                            umma_bf16(tmem_d, da + (uint64_t)(a * (A_ATOM >> 4) + 2 * k), db + (uint64_t)(a * (B_ATOM >> 4) + 2 * k), idesc,
                                      (kb > 0 || a > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(&empty[s]);                   // the stage is free once these MMAs have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[b]);                    // arrives when every MMA issued so far is complete
            }
        }
    } else {
        // epilogue: warps q and q+4 share accumulator lanes 32q … 32q+31 and take half of the columns each
        const int q = warp & 3, half = warp >> 2;
        uint32_t tc = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++tc) {
            const uint32_t b = tc & 1;
            const int m0 = SWAP ? tile * TC_BM : (tile / tiles_n) * TC_BM, n0 = SWAP ? 0 : (tile % tiles_n) * BN;
            const int m = m0 + q * 32 + lane;                 // this thread's row (when the roles are not exchanged)
            // where this thread's row goes in the cache, if the product feeds one: three loads, each waiting for
            // the one before, so they go out while the MMAs still run
            int kv_blk = -2, kv_row = 0;                      // −2: nothing to write
            if (!SWAP && kv.Kc != nullptr && m < M) {
                const int slot = kv.tok_slot[m];
                if (slot >= 0) {
                    const int pos = kv.tok_pos[m];
                    kv_blk = kv.block_table[(size_t)slot * kv.max_blocks + pos / kv.BT];
                    kv_row = pos % kv.BT;
                    if (kv_blk < 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
                }
            }
            if (*(volatile int*)s_abort || !tbar_wait_or_abort(&acc_full[b], (tc >> 1) & 1, s_abort)) { atomicExch(s_abort, 1); break; }
            if (threadIdx.x == 0) { if (tc == 0) VLRF_TRACE(trace, 3, (int)blockIdx.x, 2); VLRF_TRACE(trace, 3, (int)blockIdx.x, 3); }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + b * ACC_STRIDE + ((uint32_t)(q * 32) << 16);
            if (SWAP) {
                const int n = m0 + q * 32 + lane;             // this thread's output column = row of W
                const float bv = (bias && n < N) ? bias[n] : 0.f;
                constexpr int PER_HALF = BN >= 32 ? BN / 2 : BN;     // with 16 columns only the first half works
                if (BN >= 32 || half == 0) {
#pragma unroll 1
                    for (int c0 = half * PER_HALF; c0 < (half + 1) * PER_HALF && c0 < BN; c0 += 16) {
                        uint32_t r[16];
                        asm volatile(
                            "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                            "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                            : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                              "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                            : "r"(tmem_d + (uint32_t)c0));
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (n < N) {
                            auto rows = [&](auto act_c) {                 // the activation as a compile-time constant
                                constexpr int ACT = decltype(act_c)::value;
#pragma unroll
                                for (int j = 0; j < 16; ++j) {
                                    const int m = c0 + j;
                                    if (m < M) {
                                        float x = apply_act_const<OT, ACT>(__uint_as_float(r[j]) + bv);
                                        if (residual) x += residual[(size_t)m * ldy + n];
                                        ElemIO<OT>::store(Y + (size_t)m * ldy + n, x);
                                    }
                                }
                            };
                            if (act == VLRF_ACT_NONE) rows(std::integral_constant<int, VLRF_ACT_NONE>{});
                            else if (act == VLRF_ACT_GELU_TANH) rows(std::integral_constant<int, VLRF_ACT_GELU_TANH>{});
                            else rows(std::integral_constant<int, VLRF_ACT_GELU_ERF>{});
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) tbar_arrive(&acc_empty[b]);    // this warp has read all it needs of the accumulator
                continue;
            }
            // the two warps of a lane group share the columns in runs of 32: half and half, or 64 + 32 of 96
            constexpr int SPLIT_AT = ((BN / 32 + 1) / 2) * 32;
            const int c_begin = half ? SPLIT_AT : 0, c_end = half ? BN : SPLIT_AT;
            // whether rows of Y, and heads in the cache, lie so that 32-byte stores are aligned
            const bool wide = (reinterpret_cast<uintptr_t>(Y) & 31) == 0 && (ldy % (32 / (int)sizeof(OT))) == 0;
            const bool kv_wide = kv.Kc != nullptr && kv.dh % 16 == 0 && kv.k_off % 16 == 0 && kv.v_off % 16 == 0 &&
                                 ((reinterpret_cast<uintptr_t>(kv.Kc) | reinterpret_cast<uintptr_t>(kv.Vc)) & 31) == 0;
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_end; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + (uint32_t)c0, r);          // in flight while the bias and the residual are fetched
                const bool live = m < M && n0 + c0 < N;
                const int n_here = live ? min(32, N - (n0 + c0)) : 0;
                const bool fast = n_here == 32 && (ldy % 8) == 0;
                OT* __restrict__ yrow = Y + (size_t)m * ldy + n0 + c0;
                float4 bq[8], rq[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) { bq[i] = make_float4(0.f, 0.f, 0.f, 0.f); rq[i] = bq[i]; }
                if (fast) {
                    if (bias && ((n0 + c0) % 4 == 0)) {
#pragma unroll
                        for (int i = 0; i < 8; ++i) bq[i] = __ldg(reinterpret_cast<const float4*>(bias + n0 + c0) + i);
                    } else if (bias) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            bq[i] = make_float4(bias[n0 + c0 + 4 * i], bias[n0 + c0 + 4 * i + 1], bias[n0 + c0 + 4 * i + 2], bias[n0 + c0 + 4 * i + 3]);
                    }
                    if (residual) {
                        const float* rr = residual + (size_t)m * ldy + n0 + c0;
                        if ((reinterpret_cast<uintptr_t>(residual) & 31) == 0 && ldy % 8 == 0) {
#pragma unroll
                            for (int i = 0; i < 8; i += 2) {
                                float v8[8];
                                ld_global_32B(rr + 4 * i, v8);
                                rq[i] = make_float4(v8[0], v8[1], v8[2], v8[3]);
                                rq[i + 1] = make_float4(v8[4], v8[5], v8[6], v8[7]);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 8; ++i) rq[i] = reinterpret_cast<const float4*>(rr)[i];
                        }
                    }
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c0 + 32 >= c_end) {                       // this warp's last columns are in registers
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) tbar_arrive(&acc_empty[b]);
                }
                if (!live) continue;
                if (fast) {
                    // 16 columns at a time: 32 bytes of bfloat16 (one store where rows and heads are aligned for it),
                    // or twice 32 bytes of float32; the activation is a compile-time constant inside
                    auto fast_body = [&](auto act_c) {
                        constexpr int ACT = decltype(act_c)::value;
#pragma unroll
                        for (int j = 0; j < 32; j += 16) {
                            float v[16];
#pragma unroll
                            for (int i = 0; i < 16; i += 4) {
                                const float4 bb = bq[(j + i) / 4], rr = rq[(j + i) / 4];
                                v[i + 0] = apply_act_const<OT, ACT>(__uint_as_float(r[j + i + 0]) + bb.x) + rr.x;
                                v[i + 1] = apply_act_const<OT, ACT>(__uint_as_float(r[j + i + 1]) + bb.y) + rr.y;
                                v[i + 2] = apply_act_const<OT, ACT>(__uint_as_float(r[j + i + 2]) + bb.z) + rr.z;
                                v[i + 3] = apply_act_const<OT, ACT>(__uint_as_float(r[j + i + 3]) + bb.w) + rr.w;
                            }
                            if (sizeof(OT) == 4) {
                                float* dst = reinterpret_cast<float*>(yrow) + j;
                                if (wide) {
                                    uint32_t w0[8], w1[8];
#pragma unroll
                                    for (int i = 0; i < 8; ++i) { w0[i] = __float_as_uint(v[i]); w1[i] = __float_as_uint(v[8 + i]); }
                                    st_global_32B(dst, w0);
                                    st_global_32B(dst + 8, w1);
                                } else {
#pragma unroll
                                    for (int i = 0; i < 16; i += 4) *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                                }
                            } else {
                                uint32_t w[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i) w[i] = pack2(v[2 * i], v[2 * i + 1]);
                                __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(yrow) + j;
                                if (wide) {
                                    st_global_32B(dst, w);
                                } else {
                                    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
                                    *reinterpret_cast<uint4*>(dst + 8) = make_uint4(w[4], w[5], w[6], w[7]);
                                }
                                if (kv_blk >= 0) {
#pragma unroll
                                    for (int h8 = 0; h8 < 2; ++h8) {      // 8 columns are one head's, and one of q / k / v
                                        if (kv_wide && h8 == 1) break;   // … and so are 16, which then went out in one piece
                                        const int n = n0 + c0 + j + 8 * h8;
                                        if (n < kv.k_off) continue;
                                        const bool is_v = n >= kv.v_off;
                                        const int col = n - (is_v ? kv.v_off : kv.k_off);
                                        if (col >= kv.width) continue;
                                        const int hh = col / kv.dh, cc = col - hh * kv.dh;
                                        __nv_bfloat16* to = reinterpret_cast<__nv_bfloat16*>(is_v ? kv.Vc : kv.Kc) +
                                                            (((size_t)kv_blk * kv.Hkv + hh) * kv.BT + kv_row) * kv.dh + cc;
                                        if (kv_wide) st_global_32B(to, w);
                                        else *reinterpret_cast<uint4*>(to) = h8 ? make_uint4(w[4], w[5], w[6], w[7]) : make_uint4(w[0], w[1], w[2], w[3]);
                                    }
                                }
                            }
                        }
                    };
                    if (act == VLRF_ACT_NONE) fast_body(std::integral_constant<int, VLRF_ACT_NONE>{});
                    else if (act == VLRF_ACT_GELU_TANH) fast_body(std::integral_constant<int, VLRF_ACT_GELU_TANH>{});
                    else fast_body(std::integral_constant<int, VLRF_ACT_GELU_ERF>{});
                } else {
                    const float* rrow = residual ? residual + (size_t)m * ldy + n0 + c0 : nullptr;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {            // unrolled so that r stays in registers
                        if (j >= n_here) break;
                        float x = __uint_as_float(r[j]);
                        if (bias) x += bias[n0 + c0 + j];
                        x = apply_act_out<OT>(x, act);
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
    if (threadIdx.x == 0) VLRF_TRACE(trace, 3, (int)blockIdx.x, 6);
    // everyone meets here on every path; then the allocating warp gives the tensor memory back
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 8) {
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
    const size_t smem = 1024 + (size_t)STAGES * tc_atoms(BN) * (TC_BM * TC_BK * 2 + BN * TC_BK * 2) + (2 * STAGES + 4) * 8 + 16;
    auto kern = gemm_tcgen05_kernel<BN, STAGES, OT, SWAP>;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_tcgen05: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    const long long tiles = SWAP ? (N + TC_BM - 1) / TC_BM : (long long)((N + BN - 1) / BN) * ((M + TC_BM - 1) / TC_BM);
    const int sms = sm_count_cached();
    dim3 grid((unsigned)(tiles < sms ? tiles : sms));          // persistent: one CTA per SM at most
    cudaError_t e = launch_chained(kern, grid, dim3(TC_THREADS), smem, stream, tx, tw, bias, residual, (OT*)Y, M, N, K, ldy,
                                   act, kv, dev_err, vlrf_trace_buffer());
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_tcgen05: %s", cudaGetErrorString(e));
    return vlrf_check_launch("gemm_tcgen05");
}
}  // namespace

// A tile width (64, 96, 128, 160, 192, 224 or 256) for every product that is not given to the exchanged roles,
// instead of the choice by size; 0 gives the choice back.  For measurements.
namespace { int g_forced_width = 0; }
extern "C" int vlrf_gemm_tcgen05_force_width(int bn) {
    VLRF_REQUIRE(bn == 0 || bn == 64 || bn == 96 || bn == 128 || bn == 160 || bn == 192 || bn == 224 || bn == 256, "gemm_tcgen05: no tiles %d wide", bn);
    g_forced_width = bn;
    return VLRF_OK;
}

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
    // tile width: the fewest rounds of the persistent CTAs, each weighted by the bytes a tile's stage pulls through
    // L2 (128 rows of one operand and the tile's width of the other): that, not the MMAs, is what a round's time
    // follows when all SMs run (measured over the products of GPT-2 small to XL at 512 to 8,192 rows)
    int best_bn = 128;
    {
        const int sms = sm_count_cached();
        long long best = -1;
        const int widths[7] = {256, 224, 192, 160, 128, 96, 64};
        for (int i = 0; i < 7; ++i) {
            const int bn = widths[i];
            if (bn > 64 && N <= bn / 2) continue;
            const long long tiles = (long long)((N + bn - 1) / bn) * ((M + 127) / 128);
            const long long rounds = (tiles + sms - 1) / sms;
            if (bn == 96 && rounds > 1) continue;      // the odd width only where it puts every tile on an SM of its own
            const long long cost = rounds * (bn + 128);
            if (best < 0 || cost < best) { best = cost; best_bn = bn; }
        }
        if (g_forced_width > 0) best_bn = g_forced_width;
    }
#define TILED(BNV, ST) (out_dtype == VLRF_BF16 ? launch_tc<BNV, ST, __nv_bfloat16>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream) \
                                              : launch_tc<BNV, ST, float>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, kv, dev_err, stream))
    VLRF_REQUIRE(out_dtype == VLRF_BF16 || out_dtype == VLRF_F32, "gemm_tcgen05: unknown output dtype %d", out_dtype);
    if (best_bn == 256) return TILED(256, 4);
    if (best_bn == 224) return TILED(224, 4);
    if (best_bn == 192) return TILED(192, 5);
    if (best_bn == 160) return TILED(160, 5);
    if (best_bn == 128) return TILED(128, 3);
    if (best_bn == 96) return TILED(96, 4);
    return TILED(64, 4);
#undef TILED
}

