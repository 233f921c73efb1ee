// Y[M,N] = act(X[M,K] · W[N,K]^T + bias) (+ residual) for few rows (M ≤ 64) on the tensor cores, with the
// sum over k cut into parts: the decode step's products.
//
// Such a product reads W once and is far too little work for either roofline: what it costs is the chain of
// latencies between "the rows of X are there" and "the rows of Y are there".  A layer's matrices have only N/128
// tiles of 128 output columns, too few to keep HBM busy, so the grid is tiles × splits and the `splits` CTAs of a
// tile form a thread-block cluster: CTA (tile, s) asks for the 64-wide k blocks of part s (TMA, 128-byte swizzle; a
// ring of shared-memory stages where a part is larger than the ring) before the kernel ahead has finished, since the
// weights depend on nothing.
//
// The product itself, by the number of rows:
//   up to 16 rows (SYNC)  `mma.sync` by the CTA's warps, each on 16 (or 32) rows of the W tile read from the ring with
//       ldmatrix, times all rows of X, accumulators in registers.  One thread issuing `tcgen05.mma`, its commit, a
//       barrier and the read-back from tensor memory are the longer chain for so little work.
//   more rows  W is the 128-row operand of `tcgen05.mma`, the rows of X its N (16, 32 or 64), the accumulator in
//       tensor memory holds Yᵀ; one elected thread issues the MMAs, four warps read the accumulator back.
//
// The sum over the parts: the finished tile is dealt to the warps of all CTAs of the cluster in pieces: a row of Y by
// 32 columns up to 16 rows, four rows by 32 columns beyond.  Every thread sends each value of its partial tile (four
// rows of a column at once where pieces have four) into the shared memory of the CTA whose warp finishes the piece, as
// a store that counts down a barrier there (`st.async`): a piece crosses the cluster once, nobody waits at a cluster
// barrier or reads another CTA's memory, and a CTA leaves when it has received all it is due (which is after everyone
// stopped writing to it).
// A warp adds the parts in the order of their CTAs, so the result does not depend on timing; it then
// applies bias, GELU and the residual sum (reference include/model/feedforward.hpp:54-76,
// include/model/transformer_block.hpp:153,158), stores the piece, leaves the row statistics a later LayerNorm needs
// and, for a fused q/k/v projection, scatters K and V columns into the paged cache (reference
// include/model/kv_cache.hpp:215-251; the cache row of every token is looked up before the wait).
//
// A tile may also have 64 rows of W only (twice as many tiles for narrow matrices); with `tcgen05.mma` the MMA still
// works on 128 rows, the upper 64 being whatever follows in shared memory, and the upper 64 lanes of the
// accumulator are never read.
//
// LN: the rows of X are the float32 residual stream; eight warps compute the LayerNorm of this CTA's k range (mean
// and variance from the row statistics that the kernel which wrote the rows left; reference
// include/model/ops.hpp:443-476) and write the normalised rows as bfloat16 into shared memory in the layout TMA
// would have produced, while the weight copies are already in flight.
//
// Launched "chained": weights are requested before the kernel ahead has finished, activations only after.
// Every wait on an mbarrier is bounded; a CTA that gives up sets the device error word, sends nothing (its
// receivers then give up too, after their own bounded wait) and frees its tensor memory.
#include "common.cuh"
#include <cstdlib>
#include <cstring>
#include "tma.cuh"
#include "tcgen05.cuh"

namespace {

// warps 0-3: epilogue (and LayerNorm), 4: producer + tensor memory, 5: MMA issue, 6-9 (LN only): LayerNorm
constexpr int SP_THREADS = 192, SP_THREADS_LN = 320;
constexpr int SP_BK = 64;
constexpr int SP_MAX_STAGES = 16;
constexpr int SP_MAX_SPLITS = 16;        // the largest cluster (more than 8 is "non-portable": B200 takes it)
constexpr int SP_LN_MAX_KB = 16;         // k blocks of one part with the fused norm (a lane holds 8 float4 of a row)
constexpr int SP_STAT_SEGS = 256;        // most 32-column segments of a row whose statistics are kept (width ≤ 8192)
constexpr size_t SP_SMEM_LIMIT = 111 * 1024;   // two CTAs fit an SM: this product's and the next one's, fetching ahead

struct SpKvScatter {
    void* Kc; void* Vc;
    const int* block_table; const int* tok_slot; const int* tok_pos;
    int max_blocks, k_off, v_off, width, dh, Hkv, BT;
};

// One warp norms its CTA's k range [k_lo, k_hi) of one float32 row and writes it as bfloat16 into shared memory in
// the layout TMA would have produced (128-byte swizzle, a tile of 64 columns after the other).  JV: float4 a lane
// of the range (32 lanes × 4 columns each); JG: 32-column segments a lane of the row's statistics.  Both are
// template arguments so that a warp executes no instruction for pieces it does not have: the norm lies on the
// product's critical path and is executed by single warps, at the latency of every instruction.
// The row's mean and variance come from the per-segment sums that the kernel which wrote the row left: sum and
// squared deviation from the segment's own mean; segments combine exactly (M2 = Σ M2_g + n_g·(mean_g − mean)²),
// in a fixed order (reference include/model/ops.hpp:443-476 for the norm itself).
template <int JV, int JG>
__device__ __forceinline__ void sp_norm_row(const float* __restrict__ row, const float* __restrict__ st, int lane, int m,
                                            int k_lo, int k_hi, int K, int G, float inv_K, float eps,
                                            const float* s_gamma, const float* s_beta, unsigned char* b_tiles, int b_bytes) {
    // this CTA's k range of the row: requested first, used after the statistics
    float4 v[JV];
#pragma unroll
    for (int j = 0; j < JV; ++j) {
        const int i = k_lo + (j * 32 + lane) * 4;
        v[j] = (i < k_hi && i < K) ? *reinterpret_cast<const float4*>(row + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float sg[JG], qg[JG];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < JG; ++j) {
        const int g = j * 32 + lane;
        sg[j] = 0.f; qg[j] = 0.f;
        if (g < G) { const float2 t2 = *reinterpret_cast<const float2*>(st + 2 * g); sg[j] = t2.x; qg[j] = t2.y; }
        s += sg[j];
    }
    const float mean = warp_sum(s) * inv_K;
    float q = 0.f;
#pragma unroll
    for (int j = 0; j < JG; ++j) {
        const int g = j * 32 + lane;
        if (g < G) {
            const float n_g = (float)min(32, K - g * 32);
            const float dm = __fdividef(sg[j], n_g) - mean;
            q += qg[j] + n_g * dm * dm;
        }
    }
    const float inv = rsqrtf(warp_sum(q) * inv_K + eps);
    // normalised; columns beyond K are zeros (W reads as zeros there too)
#pragma unroll
    for (int j = 0; j < JV; ++j) {
        const int kl = (j * 32 + lane) * 4;
        const int i = k_lo + kl;
        if (i < k_hi) {
            uint2 pk = make_uint2(0u, 0u);
            if (i < K) {
                const float4 gm = *reinterpret_cast<const float4*>(s_gamma + kl);
                const float4 bt = *reinterpret_cast<const float4*>(s_beta + kl);
                pk.x = pack2((v[j].x - mean) * inv * gm.x + bt.x, (v[j].y - mean) * inv * gm.y + bt.y);
                pk.y = pack2((v[j].z - mean) * inv * gm.z + bt.z, (v[j].w - mean) * inv * gm.w + bt.w);
            }
            unsigned char* dst = b_tiles + (size_t)(kl >> 6) * b_bytes + m * 128 + ((((kl & 63) >> 3) ^ (m & 7)) << 4) + (kl & 7) * 2;
            *reinterpret_cast<uint2*>(dst) = pk;
        }
    }
}

// Floats of the buffer in which a CTA receives its warps' pieces (rp rows, 32 columns) from every part.
__host__ __device__ inline int sp_recv_floats(int M, int bm, int splits, int rp) {
    const int n_j = (((M + rp - 1) / rp) * (bm >> 5) + 4 * splits - 1) / (4 * splits);
    return splits * n_j * 4 * 32 * rp;
}
// a float into the shared memory of CTA `rank` of the cluster (at the place `own_addr` has in this CTA), counted
// down on the barrier at `own_bar`'s place there
__device__ __forceinline__ void sp_send_f32(uint32_t own_addr, uint32_t own_bar, uint32_t rank, float v) {
    uint32_t addr, bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(own_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(own_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(addr), "r"(__float_as_uint(v)), "r"(bar) : "memory");
}

__device__ __forceinline__ void sp_ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void sp_ldsm_x2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
__device__ __forceinline__ void sp_mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// SYNC: one finishing warp's product.  Its 32 rows of the W tile (two 16-row MMA tiles) times all rows of X (NT
// 8-column tiles), k block after k block from the ring; then every value is sent to whoever finishes the piece
// (row m of X, this warp's 32 columns) it is in.  An `mma.sync` has a long latency here, and the MMAs of a k block
// that add to one accumulator would wait for one another: the four 16-wide steps of a k block have accumulators of
// their own, which are added at the end (in a fixed order).
template <int NT, int MT, bool LN>
__device__ __forceinline__ bool sp_sync_product(int row0, int lane, int M, int n_kb, int stages, unsigned char* a_tiles, int a_bytes,
                                                unsigned char* b_tiles, int b_bytes, uint64_t* full, uint64_t* empty, int* s_abort,
                                                float* recv, uint64_t* recv_bar, const int* s_piece, int segs, int split, int n_j) {
    float acc[SP_BK / 16][MT][NT][4];
#pragma unroll
    for (int ks = 0; ks < SP_BK / 16; ++ks)
#pragma unroll
        for (int a = 0; a < MT; ++a)
#pragma unroll
            for (int b = 0; b < NT; ++b)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[ks][a][b][e] = 0.f;
    const int a_row = row0 + (lane & 15);                          // + 16 for a second tile
    const int b_row = (lane & 7) + ((lane >> 4) << 3);
    for (int i = 0; i < n_kb; ++i) {
        const int s = i % stages;
        if (!tbar_wait_or_abort(&full[s], (uint32_t)((i / stages) & 1), s_abort)) return false;
        const uint32_t a_base = tsm(a_tiles + (size_t)s * a_bytes), b_base = tsm(b_tiles + (size_t)(LN ? i : s) * b_bytes);
        uint32_t a[SP_BK / 16][MT][4], b[SP_BK / 16][4];
#pragma unroll
        for (int ks = 0; ks < SP_BK / 16; ++ks) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                const int row = a_row + mt * 16, ch = ks * 2 + (lane >> 4);
                sp_ldsm_x4(a_base + row * 128 + ((ch ^ (row & 7)) << 4), a[ks][mt][0], a[ks][mt][1], a[ks][mt][2], a[ks][mt][3]);
            }
            const int ch = ks * 2 + ((lane >> 3) & 1);
            if (NT == 2) sp_ldsm_x4(b_base + b_row * 128 + ((ch ^ (b_row & 7)) << 4), b[ks][0], b[ks][1], b[ks][2], b[ks][3]);
            else sp_ldsm_x2(b_base + (lane & 7) * 128 + ((ch ^ (lane & 7)) << 4), b[ks][0], b[ks][1]);
        }
#pragma unroll
        for (int ks = 0; ks < SP_BK / 16; ++ks)
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                sp_mma16816(acc[ks][mt][0], a[ks][mt][0], a[ks][mt][1], a[ks][mt][2], a[ks][mt][3], b[ks][0], b[ks][1]);
                if (NT == 2) sp_mma16816(acc[ks][mt][1], a[ks][mt][0], a[ks][mt][1], a[ks][mt][2], a[ks][mt][3], b[ks][2], b[ks][3]);
            }
        if (n_kb > stages) {                       // the stage is needed again
            __syncwarp();
            if (lane == 0) tbar_arrive(&empty[s]);
        }
    }
    const uint32_t recv0 = tsm(recv), bar0 = tsm(recv_bar);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e1 = 0; e1 < 2; ++e1) {
            const int m = nt * 8 + (lane & 3) * 2 + e1;
            if (m < M) {
                const int who = s_piece[m * segs + (row0 >> 5)], g = who & 255, j = who >> 8;
                const uint32_t base = recv0 + (uint32_t)(((split * n_j + j) * 4 + (g & 3)) * 32 + (row0 & 31) + (lane >> 2)) * 4u;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt)
#pragma unroll
                    for (int e2 = 0; e2 < 2; ++e2) {
                        const int e = e2 * 2 + e1;
                        const float v = (acc[0][mt][nt][e] + acc[1][mt][nt][e]) + (acc[2][mt][nt][e] + acc[3][mt][nt][e]);
                        sp_send_f32(base + (uint32_t)(mt * 16 + e2 * 8) * 4u, bar0, (uint32_t)(g >> 2), v);
                    }
            }
        }
    return true;
}

// four floats at once
__device__ __forceinline__ void sp_send_f32x4(uint32_t own_addr, uint32_t own_bar, uint32_t rank, float a, float b, float c, float d) {
    uint32_t addr, bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(own_addr), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(own_bar), "r"(rank));
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
                 ::"r"(addr), "r"(__float_as_uint(a)), "r"(__float_as_uint(b)), "r"(__float_as_uint(c)), "r"(__float_as_uint(d)), "r"(bar) : "memory");
}

// bm: rows of W per tile (64 or 128); stages: depth of the ring; kb_cap: most k blocks of one part
// SYNC (up to 16 rows only): the product on `mma.sync` by the CTA's warps (the eight that normed the rows, each on
// 16 rows of the W tile, or the four finishing warps, each on 32), straight from the ring (ldmatrix reads the 128-byte swizzle), the accumulators in registers: with so few
// rows an MMA is a few cycles of work, and the one thread that issues `tcgen05.mma`, its commit, the barrier and
// the read-back from tensor memory are a longer chain than eight warp-level MMAs a k block.
template <int BN, typename OT, bool LN, bool SYNC>
__global__ void __launch_bounds__(LN ? SP_THREADS_LN : SP_THREADS, 2)
gemm_splitk_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const float* __restrict__ Xf, int ldx, const float* __restrict__ gamma,
                   const float* __restrict__ beta, float eps, const float* __restrict__ bias, const float* residual,
                   OT* Y, int M, int N, int K, int ldy, int act, int bm, int stages, int kb_cap, SpKvScatter kv,
                   const float* stats_in, float* stats_out, int* __restrict__ dev_err, long long* trace) {
    extern __shared__ unsigned char sp_raw[];
    // (stations of the time stamps, kind 1: 0 the CTA begins, 1 the kernel ahead has finished, 2 the rows of X are in
    // shared memory (fused norm), 3 the products are done, 4 the partial tile is sent or in place, 5 all parts are
    // here, 6 the pieces are stored; thread 0 stamps)
    const int tcta = blockIdx.x * gridDim.y + blockIdx.y;
    if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 0);
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sp_raw) + 1023) & ~(uintptr_t)1023);
    constexpr int B_BYTES = BN * SP_BK * 2;
    constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    const int a_bytes = bm * SP_BK * 2;
    // the MMA reads 128 rows from each stage: with 64-row tiles the last stage's read runs 8 KiB further,
    // which the layout keeps inside the allocation (the B tiles follow, at least 8 KiB of them or padding)
    unsigned char* a_tiles = smem;                                   // [stages][bm][128 B]
    const int ring_bytes = stages * a_bytes;
    unsigned char* b_tiles = smem + ring_bytes + (bm == 64 ? 8192 : 0);   // LN: [kb_cap][BN][128 B], else [stages][BN][128 B]
    unsigned char* after_b = b_tiles + (size_t)(LN ? kb_cap : stages) * B_BYTES;
    float* s_gamma = reinterpret_cast<float*>(after_b);              // LN: [kb_cap·64] this part's norm weights
    float* s_beta = s_gamma + (LN ? kb_cap * SP_BK : 0);
    // what this CTA receives of the tile: the pieces its warps finish, from every part of the sum
    float* recv = s_beta + (LN ? kb_cap * SP_BK : 0);
    // The finished tile is dealt to the 4·splits finishing warps of the cluster in pieces of RP rows of Y by 32 columns
    // (RP = 1 up to 16 rows, else 4): piece u = (row group)·segs + (32-column segment) is piece u / ustride of warp
    // u % ustride of the cluster.  Every CTA sends each piece of its partial tile to the CTA whose warp finishes it, as
    // stores into that CTA's shared memory that count down a barrier there (`st.async`; with RP = 4 a thread's four
    // rows of a column in one store): recv[source part][piece of the warp j][warp][32 lanes][RP].  The receiver waits
    // on its own barrier for all the bytes it is due and adds the parts in the order of their CTAs: one crossing of the
    // cluster, no cluster barrier, and nobody's shared memory is read by another CTA.
    constexpr int RP = BN == 16 ? 1 : 4;
    const int segs = bm >> 5, units = ((M + RP - 1) / RP) * segs, ustride = 4 * (int)gridDim.y;
    static_assert(!SYNC || BN == 16, "the mma.sync variant is for up to 16 rows");
    const int n_j = (units + ustride - 1) / ustride;                     // pieces a warp
    uint64_t* full = reinterpret_cast<uint64_t*>(recv + (size_t)sp_recv_floats(M, bm, (int)gridDim.y, RP));
    uint64_t* empty = full + SP_MAX_STAGES;
    uint64_t* acc_full = empty + SP_MAX_STAGES;
    uint64_t* x_ready = acc_full + 1;
    uint64_t* recv_bar = x_ready + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(recv_bar + 1);
    int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
    int* s_kv_blk = s_abort + 1;                                     // [64]
    int* s_kv_row = s_kv_blk + 64;                                   // [64]
    int* s_piece = s_kv_row + 64;                                    // [64] (SYNC) who finishes piece u: warp of the cluster | its piece << 8

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y, splits = gridDim.y;
    const int n_kb_all = (K + SP_BK - 1) / SP_BK;
    const int kb0 = (int)(((long long)n_kb_all * split) / splits), kb1 = (int)(((long long)n_kb_all * (split + 1)) / splits);
    const int n_kb = kb1 - kb0;
    const int n0 = tile * bm;

    if (threadIdx.x == 0) {
        // (a stage is given back by the commit of its MMAs, or by every warp that read it)
        for (int s = 0; s < stages; ++s) { tbar_init(&full[s], 1); tbar_init(&empty[s], SYNC ? (uint32_t)(LN ? min(8, bm >> 4) : min(4, bm >> 5)) : 1u); }
        tbar_init(acc_full, 1);
        tbar_init(x_ready, 8);
        tbar_init(recv_bar, 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the bytes this CTA is due: its warps' pieces, once from every part
        int pieces = 0;
        for (int w = 0; w < 4; ++w)
            for (int u = split * 4 + w; u < units; u += ustride) ++pieces;
        tbar_expect_tx(recv_bar, (uint32_t)(pieces * 32 * RP * splits * 4));
    }
    // The cache's block and row of every row's token.  Positions and block tables do not come from the kernel ahead:
    // a product is let go by a product ahead of it at once, but the nearest kernel ahead that is no product (the
    // attention, the embedding) let its successors go only after its own wait, and whatever wrote positions and tables
    // (the step before's sampling kernel, copies from the host) lies before that kernel (common.cuh).
    if (kv.Kc != nullptr && (int)threadIdx.x < 64) {
        const int m = threadIdx.x;
        int blk = -2, row = 0;                                  // −2: nothing to write for this row
        if (m < M) {
            const int slot = kv.tok_slot[m];
            if (slot >= 0) {
                const int pos = kv.tok_pos[m];
                blk = kv.block_table[(size_t)slot * kv.max_blocks + pos / kv.BT];
                row = pos % kv.BT;
                if (blk < 0 && blockIdx.x == 0 && blockIdx.y == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
            }
        }
        s_kv_blk[m] = blk;
        s_kv_row[m] = row;
    }
    if (SYNC && (int)threadIdx.x < units && threadIdx.x < 64) s_piece[threadIdx.x] = ((int)threadIdx.x % ustride) | (((int)threadIdx.x / ustride) << 8);
    if (warp == 4) {
        if (lane == 0) { tma_prefetch_descriptor(&tmap_w); if (!LN) tma_prefetch_descriptor(&tmap_x); }
        __syncwarp();
        if (!SYNC) {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tsm(tmem_slot)), "r"((uint32_t)TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        } else if (lane == 0) {
            *tmem_slot = 0;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // every CTA of the cluster has set up its receiving barrier before anyone sends (waited for further down)
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

    // The weights do not depend on the kernel ahead: the first stages' tiles of W are requested at once, and
    // the norm's weights for this part's columns are copied to shared memory.
    const int first = n_kb < stages ? n_kb : stages;
    if (warp == 4 && lane == 0) {
        for (int i = 0; i < first; ++i) {
            tbar_expect_tx(&full[i], a_bytes + (LN ? 0 : B_BYTES));
            tma_load_2d(a_tiles + (size_t)i * a_bytes, &tmap_w, (kb0 + i) * SP_BK, n0, &full[i]);
        }
    }
    const bool ln_warp = LN && warp != 4 && warp != 5;
    const int lw = warp < 4 ? warp : warp - 2;                       // 0…7 among the LayerNorm warps
    if (ln_warp) {
        for (int i = lw * 32 + lane; i < n_kb * SP_BK; i += 256) {
            const int k = kb0 * SP_BK + i;
            s_gamma[i] = k < K ? gamma[k] : 0.f;
            s_beta[i] = k < K ? beta[k] : 0.f;
        }
    }
    const float inv_K = 1.f / (float)K;
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    pdl_launch_dependents();
    pdl_wait();                                    // the rows of X, the residual and the positions are ready
    if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 1);

    // pieces of the tile that this warp will finish: (row m, 32-column segment), dealt to the 4·splits
    // epilogue warps of the cluster; what the first two need from global memory is fetched now
    const int gw = split * 4 + warp;
    float pre_res[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, pre_bias[2] = {0.f, 0.f};

    if (warp == 4) {
        if (lane == 0) {
            if (!LN)
                for (int i = 0; i < first; ++i)
                    tma_load_2d(b_tiles + (size_t)i * B_BYTES, &tmap_x, (kb0 + i) * SP_BK, 0, &full[i]);
            for (int i = first; i < n_kb; ++i) {
                const int s = i % stages;
                if (!tbar_wait_or_abort(&empty[s], (uint32_t)((i / stages - 1) & 1), s_abort)) { atomicExch(s_abort, 1); break; }
                tbar_expect_tx(&full[s], a_bytes + (LN ? 0 : B_BYTES));
                tma_load_2d(a_tiles + (size_t)s * a_bytes, &tmap_w, (kb0 + i) * SP_BK, n0, &full[s]);
                if (!LN) tma_load_2d(b_tiles + (size_t)s * B_BYTES, &tmap_x, (kb0 + i) * SP_BK, 0, &full[s]);
            }
        }
    } else if (warp == 5) {
        if (!SYNC && lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(128, BN);
            bool ok = true;
            if (LN && !tbar_wait_or_abort(x_ready, 0, s_abort)) { atomicExch(s_abort, 1); ok = false; }
            for (int i = 0; i < n_kb && ok; ++i) {
                const int s = i % stages;
                if (!tbar_wait_or_abort(&full[s], (uint32_t)((i / stages) & 1), s_abort)) { atomicExch(s_abort, 1); ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc_k128(a_tiles + (size_t)s * a_bytes);
                const uint64_t db = umma_desc_k128(b_tiles + (size_t)(LN ? i : s) * B_BYTES);
#pragma unroll
                for (int k = 0; k < SP_BK / 16; ++k)
                    umma_bf16(tmem_base, da + 2 * k, db + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(acc_full);
        }
    } else {
        if (LN) {
            asm volatile("bar.sync 2, 256;" ::: "memory");     // the norm's weights are in shared memory
            const int k_lo = kb0 * SP_BK, k_hi = kb1 * SP_BK;
            const int G = (K + 31) >> 5;                       // 32-column segments of a row
            const int jv = (n_kb * SP_BK + 127) >> 7, jg = (G + 31) >> 5;        // uniform over the CTA
            for (int m = lw; m < M; m += 8) {
                const float* row = Xf + (size_t)m * ldx;
                const float* st = stats_in + (size_t)m * G * 2;
                if (jv <= 1 && jg <= 1) sp_norm_row<1, 1>(row, st, lane, m, k_lo, k_hi, K, G, inv_K, eps, s_gamma, s_beta, b_tiles, B_BYTES);
                else if (jv <= 2 && jg <= 2) sp_norm_row<2, 2>(row, st, lane, m, k_lo, k_hi, K, G, inv_K, eps, s_gamma, s_beta, b_tiles, B_BYTES);
                else if (jv <= 4 && jg <= 4) sp_norm_row<4, 4>(row, st, lane, m, k_lo, k_hi, K, G, inv_K, eps, s_gamma, s_beta, b_tiles, B_BYTES);
                else sp_norm_row<SP_LN_MAX_KB / 2, SP_STAT_SEGS / 32>(row, st, lane, m, k_lo, k_hi, K, G, inv_K, eps, s_gamma, s_beta, b_tiles, B_BYTES);
            }
            if (SYNC) {
                // every warp reads all rows: it waits for the others that normed them; then each multiplies 16 rows
                // of the W tile (an `mma.sync` is slow here, so the more warps share them the better)
                asm volatile("bar.sync 3, 256;" ::: "memory");
                if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 2);
                if (lw * 16 < bm && !*(volatile int*)s_abort) {
                    bool ok;
                    if (M > 8) ok = sp_sync_product<2, 1, LN>(lw * 16, lane, M, n_kb, stages, a_tiles, a_bytes, b_tiles, B_BYTES, full, empty,
                                                              s_abort, recv, recv_bar, s_piece, segs, split, n_j);
                    else ok = sp_sync_product<1, 1, LN>(lw * 16, lane, M, n_kb, stages, a_tiles, a_bytes, b_tiles, B_BYTES, full, empty,
                                                        s_abort, recv, recv_bar, s_piece, segs, split, n_j);
                    if (!ok) atomicExch(s_abort, 1);
                }
                if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 4);
            } else {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads these through the async proxy
                __syncwarp();
                if (lane == 0) tbar_arrive(x_ready);
            }
        }
        if (warp < 4) {
            // bias and residual of the first two pieces this warp finishes: asked for now, used at the end
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int u = gw + j * ustride;
                if (u < units) {
                    const int m0 = (u / segs) * RP, n = n0 + (u % segs) * 32 + lane;
                    if (n < N) {
                        if (bias) pre_bias[j] = bias[n];
                        if (residual) {
#pragma unroll
                            for (int e = 0; e < RP; ++e)
                                if (m0 + e < M) pre_res[j][e] = residual[(size_t)(m0 + e) * ldy + n];
                        }
                    }
                }
            }
        }
        if (SYNC && !LN && warp < 4) {
            if (warp * 32 < bm && !*(volatile int*)s_abort) {
                bool ok;
                if (M > 8) ok = sp_sync_product<2, 2, LN>(warp * 32, lane, M, n_kb, stages, a_tiles, a_bytes, b_tiles, B_BYTES, full, empty, s_abort,
                                                          recv, recv_bar, s_piece, segs, split, n_j);
                else ok = sp_sync_product<1, 2, LN>(warp * 32, lane, M, n_kb, stages, a_tiles, a_bytes, b_tiles, B_BYTES, full, empty, s_abort,
                                                    recv, recv_bar, s_piece, segs, split, n_j);
                if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 4);
                if (!ok) atomicExch(s_abort, 1);
            }
        }
        if (!SYNC && warp < 4) {
            const bool have = !*(volatile int*)s_abort && tbar_wait_or_abort(acc_full, 0, s_abort);
            if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 3);
            if (!have) atomicExch(s_abort, 1);
            float r[BN];
#pragma unroll
            for (int m = 0; m < BN; ++m) r[m] = 0.f;
            if (have && warp * 32 < bm) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t t[16];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
                        : "=r"(t[0]), "=r"(t[1]), "=r"(t[2]), "=r"(t[3]), "=r"(t[4]), "=r"(t[5]), "=r"(t[6]), "=r"(t[7]),
                          "=r"(t[8]), "=r"(t[9]), "=r"(t[10]), "=r"(t[11]), "=r"(t[12]), "=r"(t[13]), "=r"(t[14]), "=r"(t[15])
                        : "r"(taddr + (uint32_t)c0));
#pragma unroll
                    for (int j = 0; j < 16; ++j) r[c0 + j] = __uint_as_float(t[j]);
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            }
            if (have && warp * 32 < bm) {
                // this thread's column of the partial tile, RP rows at a time, to whoever finishes the piece they are in
                const uint32_t recv0 = tsm(recv), bar0 = tsm(recv_bar);
                // the piece of the first rows: its owner (a warp of the cluster, g) and which of that warp's pieces it is (j)
                int g = warp, j = 0;                       // (segs ≤ 4 ≤ ustride: one subtraction wraps)
#pragma unroll
                for (int m = 0; m < BN; m += RP) {
                    if (m < M) {
                        const int off = (((split * n_j + j) * 4 + (g & 3)) * 32 + lane) * RP;
                        if (RP == 1) sp_send_f32(recv0 + (uint32_t)off * 4u, bar0, (uint32_t)(g >> 2), r[m]);
                        else sp_send_f32x4(recv0 + (uint32_t)off * 4u, bar0, (uint32_t)(g >> 2), r[m], r[m + RP / 4], r[m + RP / 2], r[m + RP - 1]);
                        g += segs;
                        if (g >= ustride) { g -= ustride; ++j; }
                    }
                }
            }
        }
    }
    __syncwarp();
    if (!SYNC && threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 4);
    if (warp < 4 && !*(volatile int*)s_abort && !tbar_wait_or_abort(recv_bar, 0, s_abort)) atomicExch(s_abort, 1);
    if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 5);
    if (warp < 4 && !*(volatile int*)s_abort) {
        int j = 0;
        for (int u = gw; u < units; u += ustride, ++j) {
            const int m0 = (u / segs) * RP, seg0 = n0 + (u % segs) * 32, n = seg0 + lane;
            const float* mine = recv + ((size_t)(j * 4 + warp) * 32 + lane) * RP;
            float acc[RP];
#pragma unroll
            for (int e = 0; e < RP; ++e) acc[e] = 0.f;
#pragma unroll
            for (int s = 0; s < SP_MAX_SPLITS; ++s) {               // always in the order of the parts
                if (s < splits) {
                    if (RP == 4) {
                        const float4 v = *reinterpret_cast<const float4*>(mine + (size_t)s * n_j * 128 * RP);
                        acc[0] += v.x; acc[RP / 4] += v.y; acc[RP / 2] += v.z; acc[RP - 1] += v.w;
                    } else {
                        acc[0] += mine[(size_t)s * n_j * 128 * RP];
                    }
                }
            }
            const float bv = j < 2 ? (j == 0 ? pre_bias[0] : pre_bias[1]) : ((bias && n < N) ? bias[n] : 0.f);
            const int n_seg = min(32, N - seg0);
            // where this column lies in the cache, if it is a key's or a value's (the same for every row of the piece)
            __nv_bfloat16* kv_col = nullptr;
            if (n < N && kv.Kc != nullptr && n >= kv.k_off) {
                const bool is_v = n >= kv.v_off;
                const int c = n - (is_v ? kv.v_off : kv.k_off);
                if (c < kv.width) {
                    const int hh = c / kv.dh, cc = c - hh * kv.dh;
                    kv_col = reinterpret_cast<__nv_bfloat16*>(is_v ? kv.Vc : kv.Kc) + (size_t)hh * kv.BT * kv.dh + cc;
                }
            }
#pragma unroll
            for (int e = 0; e < RP; ++e) {
                const int m = m0 + e;
                if (m >= M) break;                                  // (uniform over the warp)
                float res = 0.f;
                if (j < 2) res = j == 0 ? pre_res[0][e] : pre_res[1][e];
                else if (residual && n < N) res = residual[(size_t)m * ldy + n];
                const float y = apply_act_out<OT>(acc[e] + bv, act) + res;
                if (n < N) ElemIO<OT>::store(Y + (size_t)m * ldy + n, y);
                if (stats_out != nullptr && seg0 < N) {
                    // what a LayerNorm of these rows will need: this segment's sum and squared deviation from its
                    // own mean (of the values as stored; statistics are kept of float32 rows only)
                    const float yv = n < N ? y : 0.f;
                    const float sum = warp_sum(yv);
                    const float d = n < N ? yv - sum / (float)n_seg : 0.f;
                    const float m2 = warp_sum(d * d);
                    if (lane == 0) {
                        float* so = stats_out + ((size_t)m * ((N + 31) >> 5) + (seg0 >> 5)) * 2;
                        so[0] = sum; so[1] = m2;
                    }
                }
                if (kv_col != nullptr) {
                    const int blk = s_kv_blk[m];
                    if (blk >= 0) kv_col[((size_t)blk * kv.Hkv * kv.BT + s_kv_row[m]) * kv.dh] = __float2bfloat16_rn(y);
                }
            }
        }
    }
    __syncwarp();
    if (threadIdx.x == 0) VLRF_TRACE(trace, 1, tcta, 6);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (!SYNC && warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *s_abort) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
}

int sp_sm_count() {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        sms = v > 0 ? v : 148;
    }
    return sms;
}

// Which tensor-core path a product of M ≤ 16 rows takes: `mma.sync` (measured inside whole decode steps of GPT-2
// small against `tcgen05.mma`: 0.262 against 0.302 ms at batch 1, 0.290 against 0.315 at batch 8, 0.354 against 0.369 at
// batch 16).  VLRF_B200_SPLITK_MMA=tcgen05 in the environment sends them the way of the products of more rows, =8
// those of more than 8 rows (for measurements).
bool sp_use_mma_sync(int M) {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("VLRF_B200_SPLITK_MMA");
        v = e == nullptr ? 16 : strcmp(e, "tcgen05") == 0 ? 0 : strcmp(e, "8") == 0 ? 8 : 16;
    }
    return M <= v;
}

struct SpPlan { int bm, tiles, splits, kb_cap, stages; size_t smem; };

size_t sp_smem(int bm, int bn, bool ln, int stages, int kb_cap, int M, int splits) {
    const size_t ring = (size_t)stages * bm * 128;
    const size_t part = (size_t)sp_recv_floats(M, bm, splits, bn == 16 ? 1 : 4) * sizeof(float);
    return 1024 + ring + part + (bm == 64 ? 8192 : 0) + (size_t)(ln ? kb_cap : stages) * bn * 128 +
           (ln ? (size_t)kb_cap * SP_BK * 8 : 0) + (2 * SP_MAX_STAGES + 3) * 8 + 16 + 192 * sizeof(int);
}

// Tile height, number of parts and ring depth: about one CTA per SM (so that the next product's CTAs find
// room to fetch ahead), at least one k block a part, at most the largest cluster; 64-row tiles where they
// give half as many CTAs again as 128-row tiles.
SpPlan sp_plan(int M, int N, int K, int bn, bool ln) {
    const int n_kb = (K + SP_BK - 1) / SP_BK;
    // (large matrices: a third more CTAs, i.e. fewer k blocks and MMA issues a CTA, measured to pay from about
    // 12 MB of weights on)
    const int target = (long long)N * K * 2 >= (12ll << 20) ? sp_sm_count() * 4 / 3 : sp_sm_count();
    const int max_splits = SP_MAX_SPLITS;
    const size_t limit = SP_SMEM_LIMIT;
    SpPlan best{};
    int best_ctas = -1;
    for (int bm = 128; bm >= 64; bm -= 64) {
        const int tiles = (N + bm - 1) / bm;
        int splits = (target + tiles / 2) / tiles;
        if (splits > max_splits) splits = max_splits;
        if (splits > n_kb) splits = n_kb;
        if (splits < 1) splits = 1;
        const int kb_cap = (n_kb + splits - 1) / splits;
        int stages = kb_cap < SP_MAX_STAGES ? kb_cap : SP_MAX_STAGES;
        while (stages > 1 && sp_smem(bm, bn, ln, stages, kb_cap, M, splits) > limit) --stages;
        const int ctas = tiles * splits;
        const int useful = ctas < target ? ctas : target;
        if (best_ctas < 0 || useful * 2 >= best_ctas * 3) {      // 64-row tiles only for half as many CTAs again
            best = SpPlan{bm, tiles, splits, kb_cap, stages, sp_smem(bm, bn, ln, stages, kb_cap, M, splits)};
            best_ctas = useful;
        }
    }
    return best;
}

template <int BN, typename OT, bool LN, bool SYNC>
int launch_sp_as(const void* X, const void* W, const float* gamma, const float* beta, float eps, const float* bias,
              const float* residual, void* Y, int M, int N, int K, int ldx, int ldy, int act, const SpKvScatter& kv,
              const float* stats_in, float* stats_out, int* dev_err, cudaStream_t stream) {
    const SpPlan plan = sp_plan(M, N, K, BN, LN);
    VLRF_REQUIRE(plan.smem <= 200 * 1024, "gemm_splitk: %zu bytes of shared memory", plan.smem);
    CUtensorMap tw, tx;
    int st = vlrf_make_tmap_bf16(W, N, K, K, plan.bm, SP_BK, &tw);
    if (st != VLRF_OK) return st;
    if (!LN) {
        st = vlrf_make_tmap_bf16(X, M, K, ldx, BN, SP_BK, &tx);
        if (st != VLRF_OK) return st;
    } else {
        tx = tw;   // unused
    }
    auto kern = gemm_splitk_kernel<BN, OT, LN, SYNC>;
    static bool clusters_allowed = false;
    if (!clusters_allowed) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_splitk: large clusters: %s", cudaGetErrorString(e));
        clusters_allowed = true;
    }
    static size_t allowed = 48 * 1024;
    if (plan.smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)plan.smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_splitk: %zu bytes of shared memory: %s", plan.smem, cudaGetErrorString(e));
        allowed = plan.smem;
    }
    cudaError_t e = launch_chained_cluster(kern, dim3(plan.tiles, plan.splits), dim3(LN ? SP_THREADS_LN : SP_THREADS), plan.smem,
                                           dim3(1, plan.splits, 1), stream, tw, tx, (const float*)X, ldx, gamma, beta, eps, bias, residual,
                                           (OT*)Y, M, N, K, ldy, act, plan.bm, plan.stages, plan.kb_cap, kv, stats_in, stats_out,
                                           dev_err, vlrf_trace_buffer());
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_splitk: %s", cudaGetErrorString(e));
    return vlrf_check_launch("gemm_splitk");
}
// many rows: more than four one-column pieces a warp would be a long chain of reads of the other CTAs' memory
template <int BN, typename OT, bool LN>
int launch_sp(const void* X, const void* W, const float* gamma, const float* beta, float eps, const float* bias,
              const float* residual, void* Y, int M, int N, int K, int ldx, int ldy, int act, const SpKvScatter& kv,
              const float* stats_in, float* stats_out, int* dev_err, cudaStream_t stream) {
    const SpPlan plan = sp_plan(M, N, K, BN, LN);
    if (BN == 16 && sp_use_mma_sync(M))
        return launch_sp_as<BN, OT, LN, BN == 16>(X, W, gamma, beta, eps, bias, residual, Y, M, N, K, ldx, ldy, act, kv, stats_in,
                                                 stats_out, dev_err, stream);
    return launch_sp_as<BN, OT, LN, false>(X, W, gamma, beta, eps, bias, residual, Y, M, N, K, ldx, ldy, act, kv, stats_in,
                                           stats_out, dev_err, stream);
}
}  // namespace

// Floats of the statistics of `rows` rows of `width` columns.
extern "C" long long vlrf_row_stats_floats(int rows, int width) { return (long long)rows * ((width + 31) / 32) * 2; }

// Whether this kernel takes the shape.  x_is_f32_ln: X is float32 and LayerNorm is applied to it first.
extern "C" int vlrf_gemm_splitk_takes(int M, int N, int K, int ldx, int x_is_f32_ln) {
    if (M < 1 || M > 64 || N < 1 || K < 8 || K % 8 != 0) return 0;
    if (x_is_f32_ln) {
        if (ldx % 4 != 0 || M > 16 || (K + 31) / 32 > SP_STAT_SEGS) return 0;
        return sp_plan(M, N, K, 16, true).kb_cap <= SP_LN_MAX_KB ? 1 : 0;
    }
    return ldx % 8 == 0 ? 1 : 0;
}

extern "C" int vlrf_gemm_splitk(const void* X, int x_is_f32_ln, const void* W, const float* bias, const float* residual,
                                void* Y, int out_dtype, int M, int N, int K, int ldx, int ldy, int act,
                                const float* gamma, const float* beta, float eps,
                                // optional scatter of K/V columns into the cache (Kc == nullptr: none)
                                void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                                const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT,
                                // x_is_f32_ln: the row statistics of X, [M][ceil(K/32)][2]; stats_out (or null):
                                // the same for the rows of Y, [M][ceil(N/32)][2], for a later product to use
                                const float* stats_in, float* stats_out, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_gemm_splitk_takes(M, N, K, ldx, x_is_f32_ln), "gemm_splitk: does not take M=%d N=%d K=%d ldx=%d", M, N, K, ldx);
    VLRF_REQUIRE(ldx >= K && ldy >= N && act >= 0 && act <= 2, "gemm_splitk: bad arguments");
    VLRF_REQUIRE(dev_err != nullptr, "gemm_splitk: needs the device error word");
    VLRF_REQUIRE(!x_is_f32_ln || (gamma && beta && stats_in), "gemm_splitk: the fused LayerNorm needs weight, bias and the rows' statistics");
    VLRF_REQUIRE(stats_out == nullptr || ((N + 31) / 32 <= SP_STAT_SEGS && out_dtype == VLRF_F32),
                 "gemm_splitk: statistics are kept of float32 rows of at most %d columns", SP_STAT_SEGS * 32);
    VLRF_REQUIRE(out_dtype == VLRF_BF16 || out_dtype == VLRF_F32, "gemm_splitk: unknown output dtype %d", out_dtype);
    SpKvScatter kv{};
    if (Kc != nullptr) {
        VLRF_REQUIRE(Vc && block_table && tok_slot && tok_pos && Hkv > 0 && dh > 0 && BT > 0 && max_blocks > 0,
                     "gemm_splitk: incomplete cache scatter arguments");
        VLRF_REQUIRE(out_dtype == VLRF_BF16, "gemm_splitk: the cache scatter writes bfloat16");
        kv = SpKvScatter{Kc, Vc, block_table, tok_slot, tok_pos, max_blocks, k_off, v_off, Hkv * dh, dh, Hkv, BT};
    }
#define SP_GO(BNV, LNV)                                                                                                  \
    return out_dtype == VLRF_BF16                                                                                        \
               ? launch_sp<BNV, __nv_bfloat16, LNV>(X, W, gamma, beta, eps, bias, residual, Y, M, N, K, ldx, ldy, act, kv, stats_in, stats_out, dev_err, stream) \
               : launch_sp<BNV, float, LNV>(X, W, gamma, beta, eps, bias, residual, Y, M, N, K, ldx, ldy, act, kv, stats_in, stats_out, dev_err, stream)
    if (x_is_f32_ln) { SP_GO(16, true); }
    if (M <= 16) { SP_GO(16, false); }
    if (M <= 32) { SP_GO(32, false); }
    SP_GO(64, false);
#undef SP_GO
}
