// Prompt-step attention on the tensor cores: ragged, causal, over the paged cache (bfloat16, head sizes
// 64 and 128).
//
// A CTA of four warps takes 64 consecutive new tokens of one sequence and one head; each warp owns 16 query
// rows.  The keys and values of the sequence come from its cache blocks — one 64-key block is one tile —
// by tiled TMA loads with the 128-byte swizzle into a two-stage ring, so `ldmatrix` reads them without bank
// conflicts; the query tile comes the same way from the fused q/k/v rows.  Per tile: S = Q·Kᵀ with
// `mma.sync.m16n8k16` (float32 accumulate), the causal (and window) mask on the tiles that straddle the
// diagonal, an online softmax in float32 (running max and sum per row; reference
// include/model/attention.hpp:265-307, scale :373-374, visibility k ≤ past + q :253-260, tiles beyond the
// diagonal skipped :233), P packed to bfloat16 straight from the accumulator registers, O += P·V.  The
// cache already holds this step's keys and values, so "past" and "new" keys need no distinction.
// mbarrier waits are bounded; a wait that gives up sets a bit in the device error word.
#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int PF_WARPS = 4;
constexpr int PF_BQ = 64;           // queries per CTA
constexpr int PF_BK = 64;           // keys per tile = tokens per cache block
constexpr uint32_t PF_WAIT_LIMIT = 1u << 21;

__device__ __forceinline__ uint32_t psm(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void pbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(psm(bar)), "r"(count));
}
__device__ __forceinline__ void pbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(psm(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool pbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(psm(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool pbar_wait(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < PF_WAIT_LIMIT; ++i)
        if (pbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// Address of the 16-byte piece `chunk` (0 … DH/8−1) of row `row` in a tile stored as DH/64 boxes of
// [64 rows][128 bytes], each written by TMA with the 128-byte swizzle.
template <int DH>
__device__ __forceinline__ uint32_t tile_addr(uint32_t base, int row, int chunk) {
    const int box = chunk >> 3, c = chunk & 7;
    return base + box * (64 * 128) + row * 128 + ((c ^ (row & 7)) << 4);
}

template <int DH>
__global__ void __launch_bounds__(PF_WARPS * 32)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, int q_off, const int* __restrict__ block_table,
                    int max_blocks, const int* __restrict__ seq_slot, const int* __restrict__ seq_start,
                    const int* __restrict__ seq_pos0, __nv_bfloat16* __restrict__ out, int ld_out, int H, int Hkv,
                    float scale, int window, int* __restrict__ dev_err) {
    constexpr int TILE_BYTES = 64 * DH * 2;          // one 64-row tile of Q, K or V
    constexpr int NT_S = PF_BK / 8;                  // 8-key column tiles of S
    constexpr int NT_O = DH / 8;                     // 8-wide column tiles of O
    constexpr int KS_QK = DH / 16;                   // k-steps of Q·Kᵀ
    constexpr int KS_PV = PF_BK / 16;                // k-steps of P·V
    extern __shared__ unsigned char pf_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(pf_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = smem;                                   // [64][DH]
    unsigned char* k_tiles = smem + TILE_BYTES;                     // [2][64][DH]
    unsigned char* v_tiles = k_tiles + 2 * TILE_BYTES;              // [2][64][DH]
    uint64_t* bars = reinterpret_cast<uint64_t*>(v_tiles + 2 * TILE_BYTES);   // [0]: Q, [1], [2]: stages
    __shared__ int s_bad;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int qt = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
    pdl_wait();
    pdl_launch_dependents();
    const int row0 = seq_start[seq], n_new = seq_start[seq + 1] - row0;
    if (qt * PF_BQ >= n_new) return;                 // uniform: this sequence has fewer query tiles
    const int slot = seq_slot[seq];
    if (slot < 0) return;
    const int pos0 = seq_pos0[seq];
    const int hk = h / (H / Hkv);
    const int q_first = pos0 + qt * PF_BQ;                          // absolute position of the tile's first query
    const int q_last = min(pos0 + n_new, q_first + PF_BQ) - 1;      // … and of its last
    const int kt_last = q_last / PF_BK;
    const int kt_first = (window > 0) ? max(0, q_first - window + 1) / PF_BK : 0;
    const int n_kt = kt_last - kt_first + 1;
    const int* table = block_table + (size_t)slot * max_blocks;

    if (threadIdx.x == 0) {
        s_bad = 0;
        for (int i = 0; i < 3; ++i) pbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    int n_issued = 0, n_waited = 0;                  // key/value tiles requested (thread 0) and seen landed
    auto load_kv = [&](int i) {                      // thread 0: request key/value tile number i of this CTA
        const int stage = i & 1;
        const int blk = table[kt_first + i];
        if (blk < 0) { atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK); s_bad = 1; return; }
        const int row = (blk * Hkv + hk) * PF_BK;
        pbar_expect_tx(&bars[1 + stage], 2 * TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DH / 64; ++b) {
            tma_load_2d(k_tiles + stage * TILE_BYTES + b * (64 * 128), &tmap_k, b * 64, row, &bars[1 + stage]);
            tma_load_2d(v_tiles + stage * TILE_BYTES + b * (64 * 128), &tmap_v, b * 64, row, &bars[1 + stage]);
        }
        ++n_issued;
    };
    if (threadIdx.x == 0) {
        pbar_expect_tx(&bars[0], TILE_BYTES);
#pragma unroll
        for (int b = 0; b < DH / 64; ++b)
            tma_load_2d(q_tile + b * (64 * 128), &tmap_q, q_off + h * DH + b * 64, row0 + qt * PF_BQ, &bars[0]);
        load_kv(0);
        if (n_kt > 1) load_kv(1);
    }
    __syncthreads();                                 // s_bad is known
    bool ok = !s_bad;

    // this warp's query fragments stay in registers for the whole kernel
    uint32_t qf[KS_QK][4];
    {
        const bool mine = ok ? pbar_wait(&bars[0], 0) : false;
        ok = !__syncthreads_or(!mine);               // the CTA goes on only if every thread saw the tile land
    }
    if (ok) {
        const uint32_t qb = psm(q_tile);
#pragma unroll
        for (int ks = 0; ks < KS_QK; ++ks)
            ldsm_x4(tile_addr<DH>(qb, warp * 16 + (lane & 15), ks * 2 + (lane >> 4)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
    }

    float o[NT_O][4];
#pragma unroll
    for (int j = 0; j < NT_O; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float sl2 = scale * 1.4426950408889634f;                  // scores are kept in units of log2(e)
    const int q_row[2] = {q_first + warp * 16 + g, q_first + warp * 16 + g + 8};   // absolute positions of this thread's rows

    for (int i = 0; i < n_kt; ++i) {
        const int stage = i & 1;
        const int k_base = (kt_first + i) * PF_BK;
        {
            const bool mine = ok ? pbar_wait(&bars[1 + stage], (i >> 1) & 1) : false;
            const bool all = !__syncthreads_or(!mine);
            if (ok && !all && threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
            ok = all;
            if (ok) n_waited = i + 1;
        }
        // Rows of the block behind the sequence's last token hold whatever was there before.  Their scores
        // are masked by assignment below, but 0 · V would still let a stray NaN through the MMA: clear them.
        const int valid = pos0 + n_new - k_base;      // keys of this tile that exist (uniform over the CTA)
        if (ok && valid < PF_BK) {
            unsigned char* vt = v_tiles + stage * TILE_BYTES;
            const int first_row = max(valid, 0);
            for (int idx = threadIdx.x; idx < (PF_BK - first_row) * (DH / 8); idx += PF_WARPS * 32) {
                const int row = first_row + idx / (DH / 8), chunk = idx % (DH / 8);
                *reinterpret_cast<uint4*>(vt + (chunk >> 3) * (64 * 128) + row * 128 + ((chunk & 7) << 4)) = make_uint4(0, 0, 0, 0);
            }
            __syncthreads();
        }
        if (ok) {
            const uint32_t kb = psm(k_tiles + stage * TILE_BYTES), vb = psm(v_tiles + stage * TILE_BYTES);
            float s[NT_S][4];
#pragma unroll
            for (int j = 0; j < NT_S; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < KS_QK; ks += 2) {
#pragma unroll
                for (int j = 0; j < NT_S; ++j) {
                    // matrices: (keys 8j…, k-step ks: low, high half), (same keys, k-step ks+1: low, high half)
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(tile_addr<DH>(kb, j * 8 + (lane & 7), ks * 2 + (lane >> 3)), b0, b1, b2, b3);
                    mma16816(s[j], qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], b0, b1);
                    mma16816(s[j], qf[ks + 1][0], qf[ks + 1][1], qf[ks + 1][2], qf[ks + 1][3], b2, b3);
                }
            }
            // mask what the rows may not see (only tiles that touch the diagonal or the window's edge)
            const bool need_mask = window > 0 || (k_base + PF_BK - 1 > q_first);
            float m_new[2] = {m_run[0], m_run[1]};
#pragma unroll
            for (int j = 0; j < NT_S; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    float v = s[j][e] * sl2;
                    if (need_mask) {
                        const int key = k_base + j * 8 + 2 * t + (e & 1);
                        const bool hidden = key > q_row[r] || (window > 0 && key <= q_row[r] - window);
                        if (hidden) v = -INFINITY;
                    }
                    s[j][e] = v;
                    m_new[r] = fmaxf(m_new[r], v);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 1));
                m_new[r] = fmaxf(m_new[r], __shfl_xor_sync(0xffffffffu, m_new[r], 2));
            }
            float corr[2], sum[2] = {0.f, 0.f};
#pragma unroll
            for (int r = 0; r < 2; ++r) corr[r] = (m_run[r] == -INFINITY) ? 0.f : exp2f(m_run[r] - m_new[r]);
#pragma unroll
            for (int j = 0; j < NT_S; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    const float p = (m_new[r] == -INFINITY) ? 0.f : exp2f(s[j][e] - m_new[r]);   // a row that sees nothing yet
                    s[j][e] = p;
                    sum[r] += p;
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
                sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
                l_run[r] = l_run[r] * corr[r] + sum[r];
                m_run[r] = m_new[r];
            }
#pragma unroll
            for (int j = 0; j < NT_O; ++j) { o[j][0] *= corr[0]; o[j][1] *= corr[0]; o[j][2] *= corr[1]; o[j][3] *= corr[1]; }
#pragma unroll
            for (int kk = 0; kk < KS_PV; ++kk) {
                const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]), a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
                const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int j = 0; j < NT_O; j += 2) {
                    // transposed loads: (keys 16kk…+7, dims 8j…), (keys +8…, same dims), then the same for dims 8(j+1)…
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_trans(tile_addr<DH>(vb, kk * 16 + (lane & 15), j + (lane >> 4)), b0, b1, b2, b3);
                    mma16816(o[j], a0, a1, a2, a3, b0, b1);
                    mma16816(o[j + 1], a0, a1, a2, a3, b2, b3);
                }
            }
        }
        __syncthreads();                             // every warp is done with this stage
        if (threadIdx.x == 0 && i + 2 < n_kt && !s_bad) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            load_kv(i + 2);
        }
        __syncthreads();                             // a failed lookup is known to all
        if (s_bad) ok = false;
    }
    if (!ok) {
        // leave only after the loads already requested have landed in this CTA's shared memory
        if (threadIdx.x == 0) {
            pbar_wait(&bars[0], 0);
            for (int i = n_waited; i < n_issued; ++i) pbar_wait(&bars[1 + (i & 1)], (i >> 1) & 1);
        }
        __syncthreads();
        return;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int q_local = qt * PF_BQ + warp * 16 + g + r * 8;
        if (q_local >= n_new) continue;
        const float inv = (l_run[r] > 0.f) ? 1.f / l_run[r] : 0.f;
        __nv_bfloat16* dst = out + (size_t)(row0 + q_local) * ld_out + (size_t)h * DH + 2 * t;
#pragma unroll
        for (int j = 0; j < NT_O; ++j)
            *reinterpret_cast<uint32_t*>(dst + j * 8) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
}

template <int DH>
int launch_prefill(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, long long kv_rows,
                   const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                   const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new, int H,
                   int Hkv, float scale, int window, int* dev_err, cudaStream_t stream) {
    CUtensorMap tq, tk, tv;
    int st = vlrf_make_tmap_bf16(qkv, n_tokens, ld, ld, PF_BQ, 64, &tq);
    if (st != VLRF_OK) return st;
    st = vlrf_make_tmap_bf16(Kc, kv_rows, DH, DH, PF_BK, 64, &tk);
    if (st != VLRF_OK) return st;
    st = vlrf_make_tmap_bf16(Vc, kv_rows, DH, DH, PF_BK, 64, &tv);
    if (st != VLRF_OK) return st;
    const size_t smem = 1024 + (size_t)5 * 64 * DH * 2 + 64;
    auto kern = attn_prefill_kernel<DH>;
    static bool raised = false;
    if (!raised && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_prefill: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        raised = true;
    }
    dim3 grid((max_new + PF_BQ - 1) / PF_BQ, H, n_seqs);
    cudaError_t e = launch_chained(kern, grid, dim3(PF_WARPS * 32), smem, stream, tq, tk, tv, q_off, block_table,
                                   max_blocks, seq_slot, seq_start, seq_pos0, (__nv_bfloat16*)out, ld_out, H, Hkv, scale,
                                   window, dev_err);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_prefill: %s", cudaGetErrorString(e));
    return vlrf_check_launch("attn_prefill");
}
}  // namespace

// Whether the tensor-core prompt attention takes these sizes (bfloat16 only).
extern "C" int vlrf_attn_prefill_takes(int dh, int BT, int ld, int q_off) {
    return ((dh == 64 || dh == 128) && BT == PF_BK && ld % 8 == 0 && q_off % 8 == 0) ? 1 : 0;
}

extern "C" int vlrf_attn_prefill(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                                 const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                                 const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new,
                                 int H, int Hkv, int dh, int BT, float scale, int window, int* dev_err,
                                 cudaStream_t stream) {
    VLRF_REQUIRE(vlrf_attn_prefill_takes(dh, BT, ld, q_off), "attn_prefill: head size %d / block %d / row stride %d are not taken", dh, BT, ld);
    VLRF_REQUIRE(n_tokens > 0 && n_seqs > 0 && max_new > 0 && H > 0 && Hkv > 0 && H % Hkv == 0 && max_blocks > 0, "attn_prefill: bad sizes");
    VLRF_REQUIRE(n_seqs <= 65535 && H <= 65535, "attn_prefill: too many sequences or heads for one launch");
    VLRF_REQUIRE(ld_out % 2 == 0 && window >= 0 && dev_err != nullptr, "attn_prefill: bad arguments");
    const long long kv_rows = (long long)n_blocks * Hkv * BT;
    if (dh == 64)
        return launch_prefill<64>(qkv, ld, q_off, Kc, Vc, kv_rows, block_table, max_blocks, seq_slot, seq_start, seq_pos0, out,
                                  ld_out, n_tokens, n_seqs, max_new, H, Hkv, scale, window, dev_err, stream);
    return launch_prefill<128>(qkv, ld, q_off, Kc, Vc, kv_rows, block_table, max_blocks, seq_slot, seq_start, seq_pos0, out,
                               ld_out, n_tokens, n_seqs, max_new, H, Hkv, scale, window, dev_err, stream);
}
