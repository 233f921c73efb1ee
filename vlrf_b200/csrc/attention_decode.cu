// Decode attention over the paged cache: one query per (row, head), the context split across CTAs.
//
// A decode step has few queries (rows × heads), far fewer than the GPU has SMs, and each has a long
// stream of keys and values to read; so the keys 0…position of a (row, head) are cut into `n_split`
// contiguous parts, one CTA each.  Inside a CTA four warps take the 32-key chunks of the part in turn:
// a lane computes one key's score from a 16-byte-vectorised read of its row, the warp keeps a running
// (max, sum, weighted V sum) in float32 (reference: include/model/attention.hpp:265-307), the warps'
// results are merged in shared memory, and the CTA writes its partial (max, sum, sum·V) to scratch
// memory.  The CTA that finishes a (row, head) last — found with a counter in scratch memory that it
// resets for the next call — merges the parts in the order of the splits and writes the output, so no
// second launch is needed and the result does not depend on which CTA came last.
//
// Scratch: partials float32 [rows][heads][n_split][head_dim + 2], counters int32 [rows][heads] that are
// zero between calls.  The caller provides both.
#include "common.cuh"

namespace {

template <typename ET> struct Vec16d;
template <> struct Vec16d<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec16d<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* out) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

constexpr int DEC_WARPS = 4;
constexpr int DEC_MAX_DH = 256;
constexpr int DEC_ND = DEC_MAX_DH / 32;

// DH > 0: the head size is known at compile time and everything is unrolled, with all 16-byte loads of a
// 32-key chunk in flight at once; DH == 0: any head size that is a multiple of 16, with loops.
template <typename ET, int DH>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_kernel(const ET* __restrict__ qkv, int ld, int q_off, const ET* __restrict__ Kc,
                   const ET* __restrict__ Vc, const int* __restrict__ block_table, int max_blocks,
                   const int* __restrict__ tok_slot, const int* __restrict__ tok_pos, ET* __restrict__ out,
                   int ld_out, int H, int Hkv, int dh, int BT, float scale, int window, int n_split,
                   float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ dev_err) {
    extern __shared__ float sm[];                 // q [dh] | per warp: m, l, acc[dh]
    float* q = sm;
    float* wpart = sm + dh;                       // [DEC_WARPS][dh + 2]
    __shared__ int s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    const int slot = tok_slot[row];
    if (slot < 0) return;                          // padding row: the whole CTA leaves
    const int pos = tok_pos[row];
    const int hk = h / (H / Hkv);
    const ET* qsrc = qkv + (size_t)row * ld + q_off + (size_t)h * dh;
    for (int i = threadIdx.x; i < dh; i += DEC_WARPS * 32) q[i] = ElemIO<ET>::load(qsrc + i) * scale;
    __syncthreads();

    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    const int chunk0 = first / 32;
    const int n_chunks = pos / 32 + 1 - chunk0;
    const int per_split = (n_chunks + n_split - 1) / n_split;
    const int c_begin = chunk0 + split * per_split;
    const int c_end = min(chunk0 + n_chunks, c_begin + per_split);
    const int* table = block_table + (size_t)slot * max_blocks;

    constexpr int E = 16 / (int)sizeof(ET);               // elements of a 16-byte piece
    constexpr int PARTS = DH > 0 ? DH / E : 1;            // pieces of a key's row
    constexpr int KEYS_PER_ROUND = DH > 0 ? 32 / PARTS : 1;
    constexpr int NACC = DH > 0 ? E : DEC_ND;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool lost = false;
    const int part = DH > 0 ? lane % PARTS : 0, key_in_round = DH > 0 ? lane / PARTS : 0;
    for (int c = c_begin + warp; c < c_end; c += DEC_WARPS) {
        const int k0 = c * 32;
        const int blk = table[k0 / BT];
        if (blk < 0) { lost = true; break; }
        const size_t base = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * dh;
        const int key = k0 + lane;
        const bool valid = key >= first && key <= pos;
        float s = -INFINITY;
        if (DH > 0) {
            // every lane reads its key's row (rows past the last key are inside the block: harmless, unused)
            const ET* krow = Kc + base + (size_t)lane * DH;
            float dot = 0.f;
#pragma unroll
            for (int p0 = 0; p0 < PARTS; p0 += 8) {
                float kv[8][E];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (p0 + i < PARTS) Vec16d<ET>::load(krow + (p0 + i) * E, kv[i]);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (p0 + i < PARTS) {
#pragma unroll
                        for (int j = 0; j < E; ++j) dot = fmaf(q[(p0 + i) * E + j], kv[i][j], dot);
                    }
            }
            if (valid) s = dot;
        } else if (valid) {
            const ET* krow = Kc + base + (size_t)lane * dh;
            float dot = 0.f;
            for (int cc = 0; cc < dh; cc += Vec16d<ET>::N) {
                float kv[Vec16d<ET>::N];
                Vec16d<ET>::load(krow + cc, kv);
#pragma unroll
                for (int j = 0; j < Vec16d<ET>::N; ++j) dot = fmaf(q[cc + j], kv[j], dot);
            }
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        const ET* vbase = Vc + base;
        if (DH > 0) {
            // the chunk's V rows are 32·DH contiguous elements: lane takes piece `part` of keys
            // key_in_round, key_in_round + KEYS_PER_ROUND, …
#pragma unroll
            for (int r0 = 0; r0 < PARTS; r0 += 8) {
                float vv[8][E];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (r0 + i < PARTS)
                        Vec16d<ET>::load(vbase + (size_t)((r0 + i) * KEYS_PER_ROUND + key_in_round) * DH + part * E, vv[i]);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (r0 + i < PARTS) {
                        const float pk = __shfl_sync(0xffffffffu, p, (r0 + i) * KEYS_PER_ROUND + key_in_round);
                        if (pk != 0.f) {      // keys outside the range hold whatever was there before
#pragma unroll
                            for (int j = 0; j < E; ++j) acc[j] = fmaf(pk, vv[i][j], acc[j]);
                        }
                    }
            }
        } else {
            const int n_here = min(32, pos - k0 + 1);
            for (int j = 0; j < n_here; ++j) {
                const float pj = __shfl_sync(0xffffffffu, p, j);
                if (pj == 0.f) continue;
                const ET* vrow = vbase + (size_t)j * dh;
#pragma unroll
                for (int i = 0; i < DEC_ND; ++i) {
                    const int cc = i * 32 + lane;
                    if (cc < dh) acc[i] = fmaf(pj, ElemIO<ET>::load(vrow + cc), acc[i]);
                }
            }
        }
        m = m_new;
    }
    if (lost && lane == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);

    // merge the warps of this CTA (fixed order), write the CTA's partial
    float* mine = wpart + warp * (dh + 2);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
    if (DH > 0) {
        // lanes with the same piece hold sums over different keys: add them up
#pragma unroll
        for (int o = PARTS; o < 32; o <<= 1)
#pragma unroll
            for (int j = 0; j < E; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
        if (lane < PARTS) {
#pragma unroll
            for (int j = 0; j < E; ++j) mine[2 + part * E + j] = acc[j];
        }
    } else {
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) {
            const int cc = i * 32 + lane;
            if (cc < dh) mine[2 + cc] = acc[i];
        }
    }
    __syncthreads();
    const size_t pidx = ((size_t)row * H + h) * n_split;
    if (warp == 0) {
        float M = -INFINITY;
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wpart[w * (dh + 2)]);
        float L = 0.f;
        float o[DEC_ND];
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) o[i] = 0.f;
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float* pw = wpart + w * (dh + 2);
            const float f = (pw[0] == -INFINITY) ? 0.f : expf(pw[0] - M);
            L += pw[1] * f;
#pragma unroll
            for (int i = 0; i < DEC_ND; ++i) {
                const int cc = i * 32 + lane;
                if (cc < dh) o[i] += pw[2 + cc] * f;
            }
        }
        if (n_split == 1) {
            const float inv = (L > 0.f) ? 1.f / L : 0.f;
            ET* dst = out + (size_t)row * ld_out + (size_t)h * dh;
#pragma unroll
            for (int i = 0; i < DEC_ND; ++i) {
                const int cc = i * 32 + lane;
                if (cc < dh) ElemIO<ET>::store(dst + cc, o[i] * inv);
            }
            return;
        }
        float* dstp = partials + (pidx + split) * (dh + 2);
        if (lane == 0) { dstp[0] = M; dstp[1] = L; }
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) {
            const int cc = i * 32 + lane;
            if (cc < dh) dstp[2 + cc] = o[i];
        }
        __threadfence();                           // the partial is visible before the counter moves
        __syncwarp();
        if (lane == 0) {
            const int done = atomicAdd(counters + (size_t)row * H + h, 1);
            s_last = (done == n_split - 1);
        }
    }
    if (n_split == 1) return;
    __syncthreads();
    if (!s_last || warp != 0) return;
    __threadfence();
    // this CTA finished last: merge all parts in split order
    {
        float M = -INFINITY;
        for (int s = 0; s < n_split; ++s) M = fmaxf(M, __ldcg(partials + (pidx + s) * (dh + 2)));
        float L = 0.f;
        float o[DEC_ND];
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) o[i] = 0.f;
        for (int s = 0; s < n_split; ++s) {
            const float* ps = partials + (pidx + s) * (dh + 2);
            const float pm = __ldcg(ps);
            const float f = (pm == -INFINITY) ? 0.f : expf(pm - M);
            L += __ldcg(ps + 1) * f;
#pragma unroll
            for (int i = 0; i < DEC_ND; ++i) {
                const int cc = i * 32 + lane;
                if (cc < dh) o[i] += __ldcg(ps + 2 + cc) * f;
            }
        }
        const float inv = (L > 0.f) ? 1.f / L : 0.f;
        ET* dst = out + (size_t)row * ld_out + (size_t)h * dh;
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) {
            const int cc = i * 32 + lane;
            if (cc < dh) ElemIO<ET>::store(dst + cc, o[i] * inv);
        }
        if (lane == 0) counters[(size_t)row * H + h] = 0;   // zero again for the next call
    }
}
}  // namespace

// floats of scratch for the partials and ints for the counters
extern "C" long long vlrf_attn_decode_scratch_floats(int rows, int H, int dh, int n_split) {
    return (long long)rows * H * n_split * (dh + 2);
}

extern "C" int vlrf_attn_decode(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc,
                                const int* block_table, int max_blocks, const int* tok_slot,
                                const int* tok_pos, void* out, int ld_out, int rows, int H, int Hkv, int dh,
                                int BT, float scale, int window, int n_split, float* partials, int* counters,
                                int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(rows >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "attn_decode: bad sizes");
    VLRF_REQUIRE(H % Hkv == 0, "attn_decode: %d heads cannot share %d key/value heads", H, Hkv);
    VLRF_REQUIRE(dh > 0 && dh % 16 == 0 && dh <= DEC_MAX_DH,
                 "attn_decode: head size %d is not a multiple of 16 up to %d", dh, DEC_MAX_DH);
    VLRF_REQUIRE(BT % 32 == 0, "attn_decode: cache blocks of %d tokens are not a multiple of 32", BT);
    VLRF_REQUIRE(n_split >= 1 && n_split <= 65535 && H <= 65535, "attn_decode: bad split %d", n_split);
    VLRF_REQUIRE(n_split == 1 || (partials != nullptr && counters != nullptr), "attn_decode: a split context needs scratch");
    VLRF_REQUIRE(window >= 0 && dev_err != nullptr, "attn_decode: bad window or no error word");
    if (rows == 0) return VLRF_OK;
    dim3 grid(rows, H, n_split);
    const size_t smem = (size_t)(dh + DEC_WARPS * (dh + 2)) * sizeof(float);
#define LAUNCH(ET, DHT)                                                                                      \
    attn_decode_kernel<ET, DHT><<<grid, DEC_WARPS * 32, smem, stream>>>(                                    \
        (const ET*)qkv, ld, q_off, (const ET*)Kc, (const ET*)Vc, block_table, max_blocks, tok_slot, tok_pos, \
        (ET*)out, ld_out, H, Hkv, dh, BT, scale, window, n_split, partials, counters, dev_err)
    if (dtype == VLRF_F32) {
        if (dh == 64) LAUNCH(float, 64);
        else if (dh == 128) LAUNCH(float, 128);
        else LAUNCH(float, 0);
    } else if (dtype == VLRF_BF16) {
        if (dh == 64) LAUNCH(__nv_bfloat16, 64);
        else if (dh == 128) LAUNCH(__nv_bfloat16, 128);
        else LAUNCH(__nv_bfloat16, 0);
    } else {
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "attn_decode: unknown dtype %d", dtype);
    }
#undef LAUNCH
    return vlrf_check_launch("attn_decode");
}
