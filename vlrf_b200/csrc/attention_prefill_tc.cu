// Prompt-step attention on the tcgen05 tensor cores: ragged, causal, over the paged cache (bfloat16, head
// size 64).
//
// A CTA takes 128 consecutive new tokens of one sequence and one head, and walks the sequence's keys in
// blocks of 128 (two cache blocks) up to the diagonal (reference include/model/attention.hpp:233; visibility
// k ≤ past + q :253-260; scale :373-374; softmax :265-307).  Its six warps have fixed jobs:
//   warp 4  producer: the query tile once, then key and value tiles in turn through a ring of three
//           shared-memory slots (tiled TMA loads, 128-byte swizzle, one load per 64-token cache block);
//   warp 5  one elected thread issues the MMAs: S = Q·Kᵀ (128 × 128, four k steps) into tensor memory, and,
//           once the probabilities are in shared memory, O_j = P·V (128 × 64, eight k steps; V is read as it
//           lies in the cache, head dimension contiguous, through an MN-major descriptor);
//   warps 0-3  softmax: a thread owns one query row, which is one lane of tensor memory, so the row's
//           maximum and sum need no exchange between threads.  It reads S twice with `tcgen05.ld` (maximum,
//           then exponentials), masks the blocks on the diagonal and at the window's edge, writes P as
//           bfloat16 into shared memory in the layout the MMA expects, and keeps the running maximum, the
//           sum and the 64 outputs of its row in registers: O_j of each block is read back from tensor
//           memory and added after rescaling, so tensor memory is never rescaled in place.
// Two CTAs fit an SM (96 KiB of shared memory, 256 columns of tensor memory each): while one waits for its
// MMAs the other computes exponentials.  Rows of the last cache block behind the sequence's end hold
// whatever was there before; their scores are masked by assignment and their rows of V are cleared before
// the MMA reads them (0 · NaN would not be 0).  Every wait is bounded; a CTA that gives up sets the device
// error word, waits (bounded) for its copies in flight, frees its tensor memory and leaves.
#include "common.cuh"
#include "tma.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int FT_BQ = 128, FT_BK = 128, FT_DH = 64, FT_CB = 64;   // queries / keys per block, head size, tokens per cache block
constexpr int FT_THREADS = 192;
constexpr int FT_TILE = FT_BK * FT_DH * 2;                         // bytes of a K or V tile (and of the Q tile)
constexpr int FT_SLOTS = 3;
constexpr int FT_TMEM_COLS = 256;                                  // S: columns 0-127, O_j: 128-191

// Shared-memory matrix descriptor of an MN-major tile [k][64 elements] whose rows are 128 bytes written by TMA
// with the 128-byte swizzle: the 64 elements of a row are the operand's N, rows are its K; groups of 8 rows
// are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_mn128(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((tsm(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                               // leading byte offset (one 64-wide chunk of N only): unused
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows of K
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;                               // SWIZZLE_128B
    return d;
}
// D float32, A bfloat16 K-major, B bfloat16 MN-major
__host__ __device__ constexpr uint32_t umma_idesc_bf16_bmn(int M, int N) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// 2^x for x ≤ 0 or so, in one instruction (−inf gives 0; results below the normal range are flushed to 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(FT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, int q_off, const int* __restrict__ block_table,
                       int max_blocks, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                       const int* __restrict__ seq_pos0, __nv_bfloat16* __restrict__ out, int ld_out, int H, int Hkv,
                       float scale, int window, int* __restrict__ dev_err) {
    extern __shared__ unsigned char ft_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(ft_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = smem;                                    // [128][128 B]
    unsigned char* kv_tiles = smem + FT_TILE;                        // [3][128][128 B]: K_0, V_0, K_1, V_1, … in turn
    unsigned char* p_tile = kv_tiles + FT_SLOTS * FT_TILE;           // [2][128][128 B]: keys 0-63, 64-127 of the block
    uint64_t* q_full = reinterpret_cast<uint64_t*>(p_tile + 2 * FT_TILE);
    uint64_t* full = q_full + 1;                                     // [3]
    uint64_t* empty = full + FT_SLOTS;                               // [3]
    uint64_t* s_full = empty + FT_SLOTS;
    uint64_t* p_full = s_full + 1;
    uint64_t* o_full = p_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_full + 1);
    int* s_abort = reinterpret_cast<int*>(tmem_slot + 1);
    int* s_never = s_abort + 1;                                      // stays 0: for waits that nothing calls off

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qt = gridDim.x - 1 - blockIdx.x, h = blockIdx.y, seq = blockIdx.z;     // long tiles first
    pdl_wait();
    pdl_launch_dependents();
    const int row0 = seq_start[seq], n_new = seq_start[seq + 1] - row0;
    if (qt * FT_BQ >= n_new) return;                 // uniform: this sequence has fewer query tiles
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int pos0 = seq_pos0[seq];
    const int hk = h / (H / Hkv);
    const int q_first = pos0 + qt * FT_BQ;                           // absolute position of the tile's first query
    const int q_last = min(pos0 + n_new, q_first + FT_BQ) - 1;       // … and of its last
    const int kb_last = q_last / FT_BK;
    const int kb_first = (window > 0) ? max(0, q_first - window + 1) / FT_BK : 0;
    const int n_kb = kb_last - kb_first + 1;
    const int cb_last = q_last / FT_CB;                              // last cache block that holds a visible key
    const int* table = block_table + (size_t)slot * max_blocks;

    if (threadIdx.x == 0) {
        tbar_init(q_full, 1);
        for (int i = 0; i < FT_SLOTS; ++i) { tbar_init(&full[i], 1); tbar_init(&empty[i], 1); }
        tbar_init(s_full, 1);
        tbar_init(p_full, 4);
        tbar_init(o_full, 1);
        *s_abort = 0;
        *s_never = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        if (lane == 0) { tma_prefetch_descriptor(&tmap_q); tma_prefetch_descriptor(&tmap_k); tma_prefetch_descriptor(&tmap_v); }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tsm(tmem_slot)), "r"((uint32_t)FT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = *tmem_slot, tmem_o = tmem_s + 128;

    if (warp == 4) {
        if (lane == 0) {
            tbar_expect_tx(q_full, FT_TILE);
            tma_load_2d(q_tile, &tmap_q, q_off + h * FT_DH, row0 + qt * FT_BQ, q_full);
            int n_issued = 0;                         // tiles requested: 2j is K of block j, 2j+1 its V
            bool ok = true;
            for (int t = 0; t < 2 * n_kb && ok; ++t) {
                const int sl = t % FT_SLOTS, use = t / FT_SLOTS;
                if (use >= 1 && !tbar_wait_or_abort(&empty[sl], (uint32_t)((use - 1) & 1), s_abort)) { ok = false; break; }
                const int cb0 = (kb_first + (t >> 1)) * 2;            // the block's two cache blocks
                const int n_cb = (cb0 + 1 <= cb_last) ? 2 : 1;
                int blk[2];
                for (int i = 0; i < n_cb; ++i) {
                    blk[i] = table[cb0 + i];
                    if (blk[i] < 0) { atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK); ok = false; }
                }
                if (!ok) break;
                tbar_expect_tx(&full[sl], n_cb * (FT_TILE / 2));
                for (int i = 0; i < n_cb; ++i)
                    tma_load_2d(kv_tiles + (size_t)sl * FT_TILE + i * (FT_TILE / 2), (t & 1) ? &tmap_v : &tmap_k, 0,
                                (blk[i] * Hkv + hk) * FT_CB, &full[sl]);
                ++n_issued;
            }
            if (!ok) {
                atomicExch(s_abort, 1);
                // the copies already requested land in this CTA's shared memory: wait for them before leaving
                tbar_wait_or_abort(q_full, 0, s_never);
                for (int t = max(0, n_issued - FT_SLOTS); t < n_issued; ++t)
                    tbar_wait_or_abort(&full[t % FT_SLOTS], (uint32_t)((t / FT_SLOTS) & 1), s_never);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(FT_BQ, FT_BK);
            constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(FT_BQ, FT_DH);
            bool ok = tbar_wait_or_abort(q_full, 0, s_abort);
            const uint64_t dq = umma_desc_k128(q_tile);
            for (int j = 0; j < n_kb && ok; ++j) {
                const int tk = 2 * j, tv = 2 * j + 1;
                // S_j = Q · K_jᵀ (the softmax warps have read S_{j-1}: they said so with p_full of block j-1)
                if (!tbar_wait_or_abort(&full[tk % FT_SLOTS], (uint32_t)((tk / FT_SLOTS) & 1), s_abort)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dk = umma_desc_k128(kv_tiles + (size_t)(tk % FT_SLOTS) * FT_TILE);
#pragma unroll
                for (int k = 0; k < FT_DH / 16; ++k) umma_bf16(tmem_s, dq + 2 * k, dk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                umma_commit(&empty[tk % FT_SLOTS]);
                umma_commit(s_full);
                // O_j = P_j · V_j
                if (!tbar_wait_or_abort(&full[tv % FT_SLOTS], (uint32_t)((tv / FT_SLOTS) & 1), s_abort)) { ok = false; break; }
                if (!tbar_wait_or_abort(p_full, (uint32_t)(j & 1), s_abort)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dv = umma_desc_mn128(kv_tiles + (size_t)(tv % FT_SLOTS) * FT_TILE);
#pragma unroll
                for (int k = 0; k < FT_BK / 16; ++k) {
                    // 16 keys a step: P's piece lies 32 bytes further in its 64-key half, V's 16 rows further
                    const uint64_t dp = umma_desc_k128(p_tile + (size_t)(k >> 2) * FT_TILE) + 2 * (k & 3);
                    umma_bf16(tmem_o, dp, dv + (uint64_t)(k * 16 * 128 >> 4), idesc_o, k > 0 ? 1u : 0u);
                }
                umma_commit(&empty[tv % FT_SLOTS]);
                umma_commit(o_full);
            }
            if (!ok) atomicExch(s_abort, 1);
        }
    } else {
        // ---- softmax warps: thread = query row = lane of tensor memory ----
        const int r = warp * 32 + lane;
        const int q_pos = q_first + r;
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        const float sl2 = scale * 1.4426950408889634f;               // scores in units of log2(e)
        const unsigned win_eff = window > 0 ? (unsigned)window : 0x7fffffffu;   // key visible: 0 ≤ q_pos − key < win_eff
        float o_acc[FT_DH];
#pragma unroll
        for (int d = 0; d < FT_DH; ++d) o_acc[d] = 0.f;
        float m_run = -INFINITY, l_run = 0.f, corr = 0.f;            // corr: what block j's maximum did to the sums before it
        bool ok = true;
        // O of the block before is complete (and P's buffer free): o_acc holds the blocks before that one
        // relative to the maximum before it; rescale and add
        auto add_o = [&]() {
#pragma unroll
            for (int c = 0; c < FT_DH; c += 32) {
                uint32_t ov[32];
                tmem_ld32(tmem_o + lane_addr + (uint32_t)c, ov);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) o_acc[c + i] = fmaf(o_acc[c + i], corr, __uint_as_float(ov[i]));
            }
        };
        for (int j = 0; j < n_kb; ++j) {
            const int k_base = (kb_first + j) * FT_BK;
            const bool need_mask = window > 0 || (k_base + FT_BK - 1 > q_first);     // uniform over the CTA
            if (!ok || !tbar_wait_or_abort(s_full, (uint32_t)(j & 1), s_abort)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // pass 1: the row's maximum over this block (of the raw scores: the scale is positive)
            float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
            for (int c = 0; c < FT_BK; c += 32) {
                uint32_t sv[32];
                tmem_ld32(tmem_s + lane_addr + (uint32_t)c, sv);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (need_mask) {
                    const int d0 = q_pos - (k_base + c);              // q_pos − key for i = 0
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float v = ((unsigned)(d0 - i) < win_eff) ? __uint_as_float(sv[i]) : -INFINITY;
                        mx[i & 3] = fmaxf(mx[i & 3], v);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(sv[i]));
                }
            }
            const float m_new = fmaxf(m_run, fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * sl2);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;   // a row that sees nothing yet: every p is 0
            const float corr_new = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
            if (j > 0) {
                if (!tbar_wait_or_abort(o_full, (uint32_t)((j - 1) & 1), s_abort)) { ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                add_o();
            }
            corr = corr_new;
            // pass 2: exponentials, their sum, P as bfloat16 into shared memory
            float sm4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
            for (int c = 0; c < FT_BK; c += 32) {
                uint32_t sv[32];
                tmem_ld32(tmem_s + lane_addr + (uint32_t)c, sv);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float p[32];
                if (need_mask) {
                    const int d0 = q_pos - (k_base + c);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float e = fast_exp2(fmaf(__uint_as_float(sv[i]), sl2, -m_use));
                        p[i] = ((unsigned)(d0 - i) < win_eff) ? e : 0.f;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) p[i] = fast_exp2(fmaf(__uint_as_float(sv[i]), sl2, -m_use));
                }
#pragma unroll
                for (int i = 0; i < 32; ++i) sm4[i & 3] += p[i];
                unsigned char* prow = p_tile + (size_t)(c >> 6) * FT_TILE + r * 128;
#pragma unroll
                for (int g8 = 0; g8 < 4; ++g8) {
                    uint4 pk;
                    pk.x = pack2(p[g8 * 8 + 0], p[g8 * 8 + 1]); pk.y = pack2(p[g8 * 8 + 2], p[g8 * 8 + 3]);
                    pk.z = pack2(p[g8 * 8 + 4], p[g8 * 8 + 5]); pk.w = pack2(p[g8 * 8 + 6], p[g8 * 8 + 7]);
                    const int piece = ((c & 63) >> 3) + g8;
                    *reinterpret_cast<uint4*>(prow + ((piece ^ (r & 7)) << 4)) = pk;
                }
            }
            l_run = fmaf(l_run, corr, (sm4[0] + sm4[1]) + (sm4[2] + sm4[3]));
            m_run = m_new;
            // rows of V behind the sequence's last token hold whatever was there before: clear them
            const int valid = pos0 + n_new - k_base;                  // keys of this block that exist
            if (valid < FT_BK) {
                const int tv = 2 * j + 1;
                if (!tbar_wait_or_abort(&full[tv % FT_SLOTS], (uint32_t)((tv / FT_SLOTS) & 1), s_abort)) { ok = false; break; }
                unsigned char* vt = kv_tiles + (size_t)(tv % FT_SLOTS) * FT_TILE;
                const int first_row = max(valid, 0);
                for (int idx = r; idx < (FT_BK - first_row) * 8; idx += 128)
                    *reinterpret_cast<uint4*>(vt + (first_row + (idx >> 3)) * 128 + ((idx & 7) << 4)) = make_uint4(0, 0, 0, 0);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P (and V's cleared rows) are read by the MMA
            __syncwarp();
            if (lane == 0) tbar_arrive(p_full);
        }
        if (ok && tbar_wait_or_abort(o_full, (uint32_t)((n_kb - 1) & 1), s_abort)) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            add_o();
            const int q_local = qt * FT_BQ + r;
            if (q_local < n_new) {
                const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
                __nv_bfloat16* dst = out + (size_t)(row0 + q_local) * ld_out + (size_t)h * FT_DH;
#pragma unroll
                for (int d = 0; d < FT_DH; d += 8) {
                    uint4 pk;
                    pk.x = pack2(o_acc[d] * inv, o_acc[d + 1] * inv); pk.y = pack2(o_acc[d + 2] * inv, o_acc[d + 3] * inv);
                    pk.z = pack2(o_acc[d + 4] * inv, o_acc[d + 5] * inv); pk.w = pack2(o_acc[d + 6] * inv, o_acc[d + 7] * inv);
                    *reinterpret_cast<uint4*>(dst + d) = pk;
                }
            }
        } else {
            atomicExch(s_abort, 1);
        }
    }
    // everyone meets here on every path; then the allocating warp gives the tensor memory back
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"((uint32_t)FT_TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0 && *s_abort) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
}
}  // namespace

// Whether the tcgen05 prompt attention takes these sizes (bfloat16 only): head size 64, cache blocks of 64
// tokens, rows of the output and of the fused q/k/v buffer on 16-byte boundaries.
extern "C" int vlrf_attn_prefill_tc_takes(int dh, int BT, int ld, int q_off, int ld_out) {
    return (dh == FT_DH && BT == FT_CB && ld % 8 == 0 && q_off % 8 == 0 && ld_out % 8 == 0) ? 1 : 0;
}

extern "C" int vlrf_attn_prefill_tc(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                                    const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                                    const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new,
                                    int H, int Hkv, int dh, int BT, float scale, int window, int* dev_err,
                                    cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_attn_prefill_tc_takes(dh, BT, ld, q_off, ld_out), "attn_prefill_tc: head size %d / block %d / row strides %d, %d are not taken", dh, BT, ld, ld_out);
    VLRF_REQUIRE(n_tokens > 0 && n_seqs > 0 && max_new > 0 && H > 0 && Hkv > 0 && H % Hkv == 0 && max_blocks > 0, "attn_prefill_tc: bad sizes");
    VLRF_REQUIRE(n_seqs <= 65535 && H <= 65535, "attn_prefill_tc: too many sequences or heads for one launch");
    VLRF_REQUIRE(window >= 0 && dev_err != nullptr, "attn_prefill_tc: bad arguments");
    const long long kv_rows = (long long)n_blocks * Hkv * BT;
    CUtensorMap tq, tk, tv;
    int st = vlrf_make_tmap_bf16(qkv, n_tokens, ld, ld, FT_BQ, 64, &tq);
    if (st != VLRF_OK) return st;
    st = vlrf_make_tmap_bf16(Kc, kv_rows, dh, dh, FT_CB, 64, &tk);
    if (st != VLRF_OK) return st;
    st = vlrf_make_tmap_bf16(Vc, kv_rows, dh, dh, FT_CB, 64, &tv);
    if (st != VLRF_OK) return st;
    const size_t smem = 1024 + (size_t)(1 + FT_SLOTS + 2) * FT_TILE + 16 * 8;
    static bool raised = false;
    if (!raised) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_prefill_tc: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    dim3 grid((max_new + FT_BQ - 1) / FT_BQ, H, n_seqs);
    cudaError_t e = launch_chained(attn_prefill_tc_kernel, grid, dim3(FT_THREADS), smem, stream, tq, tk, tv, q_off, block_table,
                                   max_blocks, seq_slot, seq_start, seq_pos0, (__nv_bfloat16*)out, ld_out, H, Hkv, scale,
                                   window, dev_err);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_prefill_tc: %s", cudaGetErrorString(e));
    return vlrf_check_launch("attn_prefill_tc");
}
