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
// A CTA's blocks are a chain (scores, softmax, output product, one after the other), so a step with few
// tiles is bound by its longest tile, not by the SMs' throughput.  The keys of a long tile can therefore be
// dealt to up to `n_parts` CTAs: each leaves its rows' maximum, sum and outputs in global scratch, and the
// one that finishes last (a counter per tile says which) merges all of them in a fixed order, so the result
// does not depend on which CTA that is.  Long tiles come first in the grid.
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
constexpr int FT_MIN_PART = 2;                                     // key blocks a part holds at least (what the host plans with)
constexpr int FT_PART_BLOCKS = 3;                                  // key blocks a part holds at most, while the tile has parts left
constexpr int FT_MAX_PARTS = 8;
constexpr int FT_PART_FLOATS = FT_DH * FT_BQ + 2 * FT_BQ;          // a part's scratch: outputs [64][128], maxima, sums

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

// (With 168 registers a thread an SM's four schedulers hold two CTAs of six warps only if their warps fall
// three to a scheduler, so a CTA that ends is often replaced only when its neighbour has ended too; a limit
// of 128 registers, under which any placement fits, was measured: every block became 5 % slower, which cost
// more than the waiting, since CTAs that share an SM are of similar length in the order below.)
__global__ void __launch_bounds__(FT_THREADS, 2)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                       const __grid_constant__ CUtensorMap tmap_v, int q_off, const int* __restrict__ block_table,
                       int max_blocks, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                       const int* __restrict__ seq_pos0, __nv_bfloat16* __restrict__ out, int ld_out, int H, int Hkv,
                       float scale, int window, int n_parts, float* __restrict__ partials, int* __restrict__ counters,
                       int* __restrict__ dev_err, long long* trace) {
    extern __shared__ unsigned char ft_raw[];
    // (stations of the time stamps, kind 4: 0 the CTA begins, 1 the kernel ahead has finished, 6 the CTA is done)
    const int tcta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
    if (threadIdx.x == 0) VLRF_TRACE(trace, 4, tcta, 0);
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
    int* s_last = s_never + 1;                                       // whether this CTA merges its tile's parts

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // z is the slowest index of the order in which CTAs are started: first parts before second parts, so that the
    // CTAs without work (short tiles have fewer parts) come last, and within a part long tiles first
    const int n_tiles = gridDim.z / n_parts;
    const int part = blockIdx.z / n_tiles, qt = n_tiles - 1 - blockIdx.z % n_tiles, h = blockIdx.x, seq = blockIdx.y;

    // set-up that reads nothing of the kernel ahead
    if (threadIdx.x == 0) {
        tbar_init(q_full, 1);
        for (int i = 0; i < FT_SLOTS; ++i) { tbar_init(&full[i], 1); tbar_init(&empty[i], 1); }
        tbar_init(s_full, 1);
        tbar_init(p_full, 4);
        tbar_init(o_full, 1);
        *s_abort = 0;
        *s_never = 0;
        *s_last = 1;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        if (lane == 0) { tma_prefetch_descriptor(&tmap_q); tma_prefetch_descriptor(&tmap_k); tma_prefetch_descriptor(&tmap_v); }
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tsm(tmem_slot)), "r"((uint32_t)FT_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();
    if (threadIdx.x == 0) VLRF_TRACE(trace, 4, tcta, 1);
    pdl_launch_dependents();
    const int row0 = seq_start[seq], row_end = seq_start[seq + 1], slot = seq_slot[seq], pos0 = seq_pos0[seq];
    const int n_new = row_end - row0;
    const int hk = h / (H / Hkv);
    const int q_first = pos0 + qt * FT_BQ;                           // absolute position of the tile's first query
    const int q_last = min(pos0 + n_new, q_first + FT_BQ) - 1;       // … and of its last
    const int kb_last = q_last / FT_BK;
    const int kb_first = (window > 0) ? max(0, q_first - window + 1) / FT_BK : 0;
    const int n_kb = kb_last - kb_first + 1;
    // the tile's key blocks are dealt to tile_parts CTAs; the others of its n_parts have nothing to do
    const int tile_parts = max(1, min(n_parts, (n_kb + FT_PART_BLOCKS - 1) / FT_PART_BLOCKS));
    const bool active = qt * FT_BQ < n_new && slot >= 0 && part < tile_parts;     // uniform over the CTA
    const int my_first = kb_first + part * n_kb / tile_parts;
    const int my_n = active ? kb_first + (part + 1) * n_kb / tile_parts - my_first : 0;
    const int cb_last = q_last / FT_CB;                              // last cache block that holds a visible key
    const int* table = block_table + (size_t)max(slot, 0) * max_blocks;
    const int tile_id = (seq * H + h) * n_tiles + qt;

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = *tmem_slot, tmem_o = tmem_s + 128;

    if (warp == 4) {
        if (lane == 0 && my_n > 0) {
            tbar_expect_tx(q_full, FT_TILE);
            tma_load_2d(q_tile, &tmap_q, q_off + h * FT_DH, row0 + qt * FT_BQ, q_full);
            int n_issued = 0;                         // tiles requested: 2j is K of block j, 2j+1 its V
            bool ok = true;
            for (int t = 0; t < 2 * my_n && ok; ++t) {
                const int sl = t % FT_SLOTS, use = t / FT_SLOTS;
                if (use >= 1 && !tbar_wait_or_abort(&empty[sl], (uint32_t)((use - 1) & 1), s_abort)) { ok = false; break; }
                const int cb0 = (my_first + (t >> 1)) * 2;            // the block's two cache blocks
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
        if (lane == 0 && my_n > 0) {
            constexpr uint32_t idesc_s = umma_idesc_bf16(FT_BQ, FT_BK);
            constexpr uint32_t idesc_o = umma_idesc_bf16_bmn(FT_BQ, FT_DH);
            bool ok = tbar_wait_or_abort(q_full, 0, s_abort);
            const uint64_t dq = umma_desc_k128(q_tile);
            // S_j = Q · K_jᵀ into tensor memory, four k steps
            auto issue_s = [&](int j) -> bool {
                const int tk = 2 * j;
                if (!tbar_wait_or_abort(&full[tk % FT_SLOTS], (uint32_t)((tk / FT_SLOTS) & 1), s_abort)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t dk = umma_desc_k128(kv_tiles + (size_t)(tk % FT_SLOTS) * FT_TILE);
#pragma unroll
                for (int k = 0; k < FT_DH / 16; ++k) umma_bf16(tmem_s, dq + 2 * k, dk + 2 * k, idesc_s, k > 0 ? 1u : 0u);
                umma_commit(&empty[tk % FT_SLOTS]);
                umma_commit(s_full);
                return true;
            };
            ok = ok && issue_s(0);
            for (int j = 0; j < my_n && ok; ++j) {
                // the softmax warps have read S_j and written P_j.  S_{j+1} goes first, so that they can start on
                // it while O_j = P_j · V_j is still being computed (they want O_j only after their first pass).
                if (!tbar_wait_or_abort(p_full, (uint32_t)(j & 1), s_abort)) { ok = false; break; }
                if (j + 1 < my_n && !issue_s(j + 1)) { ok = false; break; }
                const int tv = 2 * j + 1;
                if (!tbar_wait_or_abort(&full[tv % FT_SLOTS], (uint32_t)((tv / FT_SLOTS) & 1), s_abort)) { ok = false; break; }
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
    } else if (active) {
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
        for (int j = 0; j < my_n; ++j) {
            const int k_base = (my_first + j) * FT_BK;
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
        if (my_n > 0) {
            if (ok && tbar_wait_or_abort(o_full, (uint32_t)((my_n - 1) & 1), s_abort)) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                add_o();
            } else {
                ok = false;
                atomicExch(s_abort, 1);
            }
        }
        bool writes_out = true;
        if (tile_parts > 1) {
            // leave this part's result in scratch ([d][row], so that a warp writes whole lines), then see
            // whether the tile's other parts are all there
            float* mine = partials + ((size_t)tile_id * n_parts + part) * FT_PART_FLOATS;
#pragma unroll
            for (int d = 0; d < FT_DH; ++d) mine[d * FT_BQ + r] = o_acc[d];
            mine[FT_DH * FT_BQ + r] = m_run;
            mine[FT_DH * FT_BQ + FT_BQ + r] = l_run;
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (r == 0) {
                const int before = atomicAdd(&counters[tile_id], 1);
                *s_last = (before == tile_parts - 1) ? 1 : 0;
                if (before == tile_parts - 1) counters[tile_id] = 0;          // left as it was found
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            writes_out = *s_last != 0;
            if (writes_out) {
                __threadfence();
                // every part in turn, this CTA's own included: the sum does not depend on who came last
                m_run = -INFINITY; l_run = 0.f;
#pragma unroll
                for (int d = 0; d < FT_DH; ++d) o_acc[d] = 0.f;
                for (int p = 0; p < tile_parts; ++p) {
                    const float* theirs = partials + ((size_t)tile_id * n_parts + p) * FT_PART_FLOATS;
                    const float m_p = __ldcg(theirs + FT_DH * FT_BQ + r), l_p = __ldcg(theirs + FT_DH * FT_BQ + FT_BQ + r);
                    const float m_new = fmaxf(m_run, m_p);
                    const float a = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);
                    const float b = (m_p == -INFINITY) ? 0.f : fast_exp2(m_p - m_new);
                    l_run = fmaf(l_run, a, l_p * b);
                    m_run = m_new;
#pragma unroll
                    for (int d0 = 0; d0 < FT_DH; d0 += 16) {
                        float v[16];
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __ldcg(theirs + (d0 + i) * FT_BQ + r);
#pragma unroll
                        for (int i = 0; i < 16; ++i) o_acc[d0 + i] = fmaf(o_acc[d0 + i], a, v[i] * b);
                    }
                }
            }
        }
        if (writes_out && ok) {
            // the row as bfloat16 into shared memory (P's tile: no MMA reads it any more), then each warp
            // writes its 32 rows four at a time, so that a store instruction fills whole lines
            const float inv = (l_run > 0.f) ? 1.f / l_run : 0.f;
            unsigned char* stage = p_tile;                            // [128][128 B], 16-byte pieces swizzled by row
#pragma unroll
            for (int d = 0; d < FT_DH; d += 8) {
                uint4 pk;
                pk.x = pack2(o_acc[d] * inv, o_acc[d + 1] * inv); pk.y = pack2(o_acc[d + 2] * inv, o_acc[d + 3] * inv);
                pk.z = pack2(o_acc[d + 4] * inv, o_acc[d + 5] * inv); pk.w = pack2(o_acc[d + 6] * inv, o_acc[d + 7] * inv);
                *reinterpret_cast<uint4*>(stage + r * 128 + ((((d >> 3)) ^ (r & 7)) << 4)) = pk;
            }
            __syncwarp();
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int rr = warp * 32 + it * 4 + (lane >> 3), piece = lane & 7;
                const int q_local = qt * FT_BQ + rr;
                if (q_local < n_new) {
                    const uint4 pk = *reinterpret_cast<const uint4*>(stage + rr * 128 + ((piece ^ (rr & 7)) << 4));
                    *reinterpret_cast<uint4*>(out + (size_t)(row0 + q_local) * ld_out + (size_t)h * FT_DH + piece * 8) = pk;
                }
            }
        }
    }
    // everyone meets here on every path; then the allocating warp gives the tensor memory back
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"((uint32_t)FT_TMEM_COLS) : "memory");
    }
    if (threadIdx.x == 0) VLRF_TRACE(trace, 4, tcta, 6);
    if (threadIdx.x == 0 && *s_abort) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
}
}  // namespace

// Whether the tcgen05 prompt attention takes these sizes (bfloat16 only): head size 64, cache blocks of 64
// tokens, rows of the output and of the fused q/k/v buffer on 16-byte boundaries.
extern "C" int vlrf_attn_prefill_tc_takes(int dh, int BT, int ld, int q_off, int ld_out) {
    return (dh == FT_DH && BT == FT_CB && ld % 8 == 0 && q_off % 8 == 0 && ld_out % 8 == 0) ? 1 : 0;
}

// Scratch of one part of a tile, in floats; the most parts a tile is dealt to; key blocks (of 128) a part holds
// at least; queries of a tile.
extern "C" int vlrf_attn_prefill_tc_part_floats() { return FT_PART_FLOATS; }
extern "C" int vlrf_attn_prefill_tc_max_parts() { return FT_MAX_PARTS; }
extern "C" int vlrf_attn_prefill_tc_min_part_blocks() { return FT_MIN_PART; }
extern "C" int vlrf_attn_prefill_tc_tile() { return FT_BQ; }

// n_parts > 1 wants `partials` ([sequences × heads × tiles × n_parts] × part_floats) and `counters`
// ([sequences × heads × tiles], zero; left zero).
extern "C" int vlrf_attn_prefill_tc(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                                    const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                                    const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new,
                                    int H, int Hkv, int dh, int BT, float scale, int window, int n_parts, float* partials,
                                    int* counters, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_attn_prefill_tc_takes(dh, BT, ld, q_off, ld_out), "attn_prefill_tc: head size %d / block %d / row strides %d, %d are not taken", dh, BT, ld, ld_out);
    VLRF_REQUIRE(n_tokens > 0 && n_seqs > 0 && max_new > 0 && H > 0 && Hkv > 0 && H % Hkv == 0 && max_blocks > 0, "attn_prefill_tc: bad sizes");
    VLRF_REQUIRE(n_seqs <= 65535, "attn_prefill_tc: too many sequences for one launch");
    VLRF_REQUIRE(window >= 0 && dev_err != nullptr, "attn_prefill_tc: bad arguments");
    VLRF_REQUIRE(n_parts >= 1 && n_parts <= FT_MAX_PARTS && (n_parts == 1 || (partials != nullptr && counters != nullptr)),
                 "attn_prefill_tc: %d parts (1 to %d; more than one wants scratch)", n_parts, FT_MAX_PARTS);
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
    const long long tiles = (max_new + FT_BQ - 1) / FT_BQ;
    VLRF_REQUIRE(tiles * n_parts <= 65535, "attn_prefill_tc: %lld tiles of %d parts are too many for one launch", tiles, n_parts);
    dim3 grid(H, n_seqs, (unsigned)(tiles * n_parts));
    cudaError_t e = launch_chained(attn_prefill_tc_kernel, grid, dim3(FT_THREADS), smem, stream, tq, tk, tv, q_off, block_table,
                                   max_blocks, seq_slot, seq_start, seq_pos0, (__nv_bfloat16*)out, ld_out, H, Hkv, scale,
                                   window, n_parts, partials, counters, dev_err, vlrf_trace_buffer());
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_prefill_tc: %s", cudaGetErrorString(e));
    return vlrf_check_launch("attn_prefill_tc");
}
