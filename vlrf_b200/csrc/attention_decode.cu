// Decode attention over the paged cache: one query per (row, head), the context split across CTAs.
//
// A decode step has few queries (rows × heads), far fewer than the GPU has SMs, and each has a long
// stream of keys and values to read; so the keys 0…position of a (row, head) are cut into `n_split`
// contiguous parts, one CTA each.  Inside a CTA eight warps take the 32-key chunks of the part in turn
// and each keeps a running (max, sum, weighted V sum) in float32 (reference:
// include/model/attention.hpp:265-307); the warps' results are merged in shared memory, and the CTA
// writes its partial (max, sum, sum·V) to scratch memory.  For head sizes 64 and 128 the keys and values
// come by bulk copies into shared memory, all of a part in flight at once, on bounded mbarrier waits.  The CTA that finishes a (row, head) last — found with a counter in scratch memory that it
// resets for the next call — merges the parts in the order of the splits and writes the output, so no
// second launch is needed and the result does not depend on which CTA came last.
//
// Scratch: partials float32 [rows][heads][n_split][head_dim + 2], counters int32 [rows][heads] that are
// zero between calls.  The caller provides both.
#include "common.cuh"
#include "tma.cuh"

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

constexpr int DEC_WARPS = 8;
constexpr int DEC_MAX_DH = 256;
constexpr int DEC_ND = DEC_MAX_DH / 32;
constexpr uint32_t DEC_WAIT_LIMIT = 4000000u;
constexpr int DEC_STAGE_BYTES = 64 * 1024;       // shared memory for the keys and values in flight
constexpr int DEC_MAX_CLUSTER = 16;              // CTAs of a cluster (more than 8 is "non-portable": B200 takes it)

__device__ __forceinline__ uint32_t dsmem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void dmbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(dsmem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void dmbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(dsmem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool dmbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(dsmem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void dbulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dsmem_u32(dst)), "l"(src), "r"(bytes), "r"(dsmem_u32(bar)) : "memory");
}

// What every variant does once its warps hold (m, l, acc by dimension) in `wpart` [DEC_WARPS][dh + 2]:
// merge the warps in order, write the output (one split) or the CTA's partial, and let the CTA that
// finishes a (row, head) last merge all splits in order.
template <typename ET>
__device__ void finish_cta(const float* wpart, int dh, int row, int h, int H, int split, int n_split,
                           float* __restrict__ partials, int* __restrict__ counters, ET* __restrict__ out,
                           int ld_out, int* s_last) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
            *s_last = (done == n_split - 1);
        }
    }
    if (n_split == 1) return;
    __syncthreads();
    if (!*s_last || warp != 0) return;
    __threadfence();
    // this CTA finished last: merge all parts in split order
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

// Any head size that is a multiple of 16: ordinary loads, loops over the head size.
// The same end for CTAs launched as a cluster over the parts of one (row, head): every CTA leaves the merge of
// its warps in its own shared memory (`cpart`, dh + 2 floats), and after a cluster barrier the CTA of part 0
// reads them all through distributed shared memory and merges them in the order of the parts.  No scratch in
// global memory, no counter.  Every thread of every CTA of the cluster must come here.
template <typename ET>
__device__ void finish_cluster(const float* wpart, float* cpart, int dh, int row, int h, int split, int n_split,
                               ET* __restrict__ out, int ld_out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
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
        if (lane == 0) { cpart[0] = M; cpart[1] = L; }
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) {
            const int cc = i * 32 + lane;
            if (cc < dh) cpart[2 + cc] = o[i];
        }
    }
    cluster_sync_all();                            // every part's merge is in its CTA's shared memory
    if (split == 0 && warp == 0) {
        const uint32_t base = (uint32_t)__cvta_generic_to_shared(cpart);
        float M = -INFINITY;
        for (int s = 0; s < n_split; ++s) M = fmaxf(M, ld_cluster_f32(base, (uint32_t)s));
        float L = 0.f;
        float o[DEC_ND];
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) o[i] = 0.f;
        for (int s = 0; s < n_split; ++s) {
            const float pm = ld_cluster_f32(base, (uint32_t)s);
            const float f = (pm == -INFINITY) ? 0.f : expf(pm - M);
            L += ld_cluster_f32(base + 4, (uint32_t)s) * f;
#pragma unroll
            for (int i = 0; i < DEC_ND; ++i) {
                const int cc = i * 32 + lane;
                if (cc < dh) o[i] += ld_cluster_f32(base + 4 * (2 + cc), (uint32_t)s) * f;
            }
        }
        const float inv = (L > 0.f) ? 1.f / L : 0.f;
        ET* dst = out + (size_t)row * ld_out + (size_t)h * dh;
#pragma unroll
        for (int i = 0; i < DEC_ND; ++i) {
            const int cc = i * 32 + lane;
            if (cc < dh) ElemIO<ET>::store(dst + cc, o[i] * inv);
        }
    }
    cluster_sync_relaxed();                        // nobody leaves while its shared memory is being read
}

// The same end without a cluster barrier: every CTA of the cluster sends the merge of its warps (maximum, sum,
// outputs: dh + 2 floats) into the shared memory of the CTA of part 0, `crecv` [n_split][dh + 2], as stores that
// count down the barrier `cbar` there (`st.async`); that CTA waits for all the bytes it is due and merges the parts
// in their order.  The others leave as soon as they have sent.  Before anyone sends, every CTA has initialised its
// barrier (the CTA of part 0 expecting n_split · (dh + 2) floats) and met the others at a cluster barrier.
template <typename ET, int DH>
__device__ __forceinline__ void finish_cluster_push(const float* wpart, float* crecv, uint64_t* cbar, int row, int h, int split,
                                                    int n_split, ET* __restrict__ out, int ld_out, int* __restrict__ dev_err) {
    constexpr int ND = DH / 32;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp != 0) return;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wpart[w * (DH + 2)]);
    float L = 0.f;
    float o[ND];
#pragma unroll
    for (int i = 0; i < ND; ++i) o[i] = 0.f;
#pragma unroll
    for (int w = 0; w < DEC_WARPS; ++w) {
        const float* pw = wpart + w * (DH + 2);
        const float f = (pw[0] == -INFINITY) ? 0.f : expf(pw[0] - M);
        L += pw[1] * f;
#pragma unroll
        for (int i = 0; i < ND; ++i) o[i] += pw[2 + i * 32 + lane] * f;
    }
    {
        uint32_t dst, bar;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(dsmem_u32(crecv + (size_t)split * (DH + 2))), "r"(0));
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(dsmem_u32(cbar)), "r"(0));
        if (lane == 0) {
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(dst), "r"(__float_as_uint(M)), "r"(bar) : "memory");
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(dst + 4u), "r"(__float_as_uint(L)), "r"(bar) : "memory");
        }
#pragma unroll
        for (int i = 0; i < ND; ++i)
            asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];" ::"r"(dst + 4u * (uint32_t)(2 + i * 32 + lane)), "r"(__float_as_uint(o[i])), "r"(bar) : "memory");
    }
    if (split != 0) return;
    uint32_t polls = 0;
    while (!dmbar_try_wait(cbar, 0)) {
        if (++polls > DEC_WAIT_LIMIT) { if (lane == 0) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT); return; }
    }
    // all parts are here: merge them in their order (four at a time, so that the reads do not wait for one another)
    float Mx = -INFINITY;
    for (int s = 0; s < n_split; ++s) Mx = fmaxf(Mx, crecv[(size_t)s * (DH + 2)]);
    float Lx = 0.f;
#pragma unroll
    for (int i = 0; i < ND; ++i) o[i] = 0.f;
    for (int s = 0; s < n_split; ++s) {
        const float* ps = crecv + (size_t)s * (DH + 2);
        const float f = (ps[0] == -INFINITY) ? 0.f : expf(ps[0] - Mx);
        Lx += ps[1] * f;
#pragma unroll
        for (int i = 0; i < ND; ++i) o[i] += ps[2 + i * 32 + lane] * f;
    }
    const float inv = (Lx > 0.f) ? 1.f / Lx : 0.f;
    ET* dst = out + (size_t)row * ld_out + (size_t)h * DH;
#pragma unroll
    for (int i = 0; i < ND; ++i) ElemIO<ET>::store(dst + i * 32 + lane, o[i] * inv);
}

template <typename ET>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_generic_kernel(const ET* __restrict__ qkv, int ld, int q_off, const ET* __restrict__ Kc,
                           const ET* __restrict__ Vc, const int* __restrict__ block_table, int max_blocks,
                           const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                           ET* __restrict__ out, int ld_out, int H, int Hkv, int dh, int BT, float scale,
                           int window, int n_split, float* __restrict__ partials, int* __restrict__ counters,
                           int* __restrict__ dev_err) {
    extern __shared__ float sm[];                 // q [dh] | per warp: m, l, acc[dh]
    float* q = sm;
    float* wpart = sm + dh;                       // [DEC_WARPS][dh + 2]
    __shared__ int s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    pdl_wait();                                    // everything read below was written by earlier kernels
    pdl_launch_dependents();                       // the next kernel may start fetching its weights
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

    float acc[DEC_ND];
#pragma unroll
    for (int i = 0; i < DEC_ND; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool lost = false;
    for (int c = c_begin + warp; c < c_end; c += DEC_WARPS) {
        const int k0 = c * 32;
        const int blk = table[k0 / BT];
        if (blk < 0) { lost = true; break; }
        const size_t base = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * dh;
        const int key = k0 + lane;
        const bool valid = key >= first && key <= pos;
        float s = -INFINITY;
        if (valid) {
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
        for (int i = 0; i < DEC_ND; ++i) acc[i] *= corr;
        const int n_here = min(32, pos - k0 + 1);
        const ET* vbase = Vc + base;
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
        m = m_new;
    }
    if (lost && lane == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
    float* mine = wpart + warp * (dh + 2);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
    for (int i = 0; i < DEC_ND; ++i) {
        const int cc = i * 32 + lane;
        if (cc < dh) mine[2 + cc] = acc[i];
    }
    __syncthreads();
    finish_cta<ET>(wpart, dh, row, h, H, split, n_split, partials, counters, out, ld_out, &s_last);
}

// Head size known at compile time.  The keys and values of the CTA's part are fetched by bulk copies,
// 32 keys (one contiguous piece of a cache block) per copy, all in flight at once, each chunk completing on
// its own mbarrier.  A 16-byte piece of a key's row belongs to one lane: the PARTS lanes of a key add
// their partial dot products with shuffles, and the same lanes then weigh the same key's value pieces,
// so a quarter warp always reads 128 contiguous bytes of shared memory.
// CLUSTER: the CTAs of one (row, head) — grid z — are a thread-block cluster and merge through shared memory
template <typename ET, int DH, bool CLUSTER>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_bulk_kernel(const ET* __restrict__ qkv, int ld, int q_off, const ET* __restrict__ Kc,
                        const ET* __restrict__ Vc, const int* __restrict__ block_table, int max_blocks,
                        const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                        ET* __restrict__ out, int ld_out, int H, int Hkv, int BT, float scale, int window,
                        int n_split, float* __restrict__ partials, int* __restrict__ counters,
                        int* __restrict__ dev_err) {
    constexpr int E = 16 / (int)sizeof(ET);               // elements of a 16-byte piece
    constexpr int PARTS = DH / E;                         // pieces of a key's row = lanes per key
    constexpr int KPR = 32 / PARTS;                       // keys per round of 32 lanes
    constexpr int ROUNDS = PARTS;                         // rounds per 32-key chunk
    constexpr int CHUNK_BYTES = 32 * DH * (int)sizeof(ET);
    constexpr int CH_MAX = DEC_STAGE_BYTES / (2 * CHUNK_BYTES) < 8 ? DEC_STAGE_BYTES / (2 * CHUNK_BYTES) : 8;
    static_assert(CH_MAX >= 1, "stage too small");
    extern __shared__ __align__(128) unsigned char dsm[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(dsm);                        // CH_MAX barriers
    unsigned char* kbuf = dsm + 128;                                         // [CH_MAX][CHUNK_BYTES]
    unsigned char* vbuf = kbuf + (size_t)CH_MAX * CHUNK_BYTES;
    float* wpart = reinterpret_cast<float*>(vbuf + (size_t)CH_MAX * CHUNK_BYTES);   // [DEC_WARPS][DH + 2]
    float* cpart = wpart + DEC_WARPS * (DH + 2);                                    // [DH + 2] (CLUSTER)
    __shared__ int s_last;
    __shared__ int s_bad;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    // Before the wait: positions, tables and the cache of earlier positions come from kernels before the one
    // ahead (every kernel lets its successor begin only after its own wait), so the first chunks of keys and
    // values are requested at once.  Only the chunk that holds the new position is written by the kernel
    // ahead; it is requested after the wait, like the query.
    const int slot = tok_slot[row];
    if (slot < 0) return;                          // padding row: the whole CTA leaves
    const int pos = tok_pos[row];
    const int hk = h / (H / Hkv);
    const int part = lane % PARTS, kir = lane / PARTS;

    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    const int chunk0 = first / 32;
    const int n_chunks = pos / 32 + 1 - chunk0;
    const int per_split = (n_chunks + n_split - 1) / n_split;
    const int c_begin = chunk0 + split * per_split;
    const int c_end = min(chunk0 + n_chunks, c_begin + per_split);
    const int c_new = pos / 32;                    // the chunk with the key that the kernel ahead writes
    const int* table = block_table + (size_t)slot * max_blocks;

    if (threadIdx.x == 0) {
        s_bad = 0;
        for (int i = 0; i < CH_MAX; ++i) dmbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // thread i requests chunk r0 + i of a round into buffer i
    auto request = [&](int r0) -> bool {
        const int k0 = (r0 + threadIdx.x) * 32;
        const int blk = table[k0 / BT];
        if (blk < 0) {
            atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
            s_bad = 1;
            return false;
        }
        const size_t base = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * DH;
        dmbar_expect_tx(&bars[threadIdx.x], 2 * CHUNK_BYTES);
        dbulk_g2s(kbuf + (size_t)threadIdx.x * CHUNK_BYTES, Kc + base, CHUNK_BYTES, &bars[threadIdx.x]);
        dbulk_g2s(vbuf + (size_t)threadIdx.x * CHUNK_BYTES, Vc + base, CHUNK_BYTES, &bars[threadIdx.x]);
        return true;
    };
    bool issued = false;
    if ((int)threadIdx.x < min(CH_MAX, c_end - c_begin) && c_begin + (int)threadIdx.x != c_new) issued = request(c_begin);
    pdl_wait();                                    // the new key and value and the query are written
    pdl_launch_dependents();
    // this lane's piece of the query, scaled
    float q[E];
    {
        const ET* qsrc = qkv + (size_t)row * ld + q_off + (size_t)h * DH + part * E;
#pragma unroll
        for (int j = 0; j < E; ++j) q[j] = ElemIO<ET>::load(qsrc + j) * scale;
    }

    float acc[E];
#pragma unroll
    for (int j = 0; j < E; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool gave_up = false;
    uint32_t parity = 0;
    for (int r0 = c_begin; r0 < c_end; r0 += CH_MAX) {
        const int n_here = min(CH_MAX, c_end - r0);
        if (r0 > c_begin) {
            issued = false;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // reads of the buffers before refilling them
        }
        if ((int)threadIdx.x < n_here && (r0 > c_begin || r0 + (int)threadIdx.x == c_new)) issued = request(r0);
        __syncthreads();                           // s_bad is known
        if (s_bad) {                               // leave only after the copies already issued have landed
            if (issued) {
                uint32_t polls = 0;
                while (!dmbar_try_wait(&bars[threadIdx.x], parity) && ++polls <= DEC_WAIT_LIMIT) {}
            }
            __syncthreads();
            break;
        }
        for (int i = warp; i < n_here && !gave_up; i += DEC_WARPS) {
            uint32_t polls = 0;
            while (!dmbar_try_wait(&bars[i], parity)) {
                if (++polls > DEC_WAIT_LIMIT) { gave_up = true; break; }
            }
            if (gave_up) break;
            const int k0 = (r0 + i) * 32;
            const ET* kc = reinterpret_cast<const ET*>(kbuf + (size_t)i * CHUNK_BYTES);
            const ET* vc = reinterpret_cast<const ET*>(vbuf + (size_t)i * CHUNK_BYTES);
            float s[ROUNDS];
#pragma unroll
            for (int r = 0; r < ROUNDS; ++r) {
                float kv[E];
                Vec16d<ET>::load(kc + (size_t)(r * KPR + kir) * DH + part * E, kv);
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < E; ++j) d = fmaf(q[j], kv[j], d);
                s[r] = d;
            }
            float cmax = -INFINITY;
#pragma unroll
            for (int r = 0; r < ROUNDS; ++r) {
#pragma unroll
                for (int o = 1; o < PARTS; o <<= 1) s[r] += __shfl_xor_sync(0xffffffffu, s[r], o);
                const int key = k0 + r * KPR + kir;
                if (key < first || key > pos) s[r] = -INFINITY;
                cmax = fmaxf(cmax, s[r]);
            }
#pragma unroll
            for (int o = PARTS; o < 32; o <<= 1) cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
            const float m_new = fmaxf(m, cmax);            // a chunk that is visited has a visible key
            const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < E; ++j) acc[j] *= corr;
#pragma unroll
            for (int r = 0; r < ROUNDS; ++r) {
                const float p = (s[r] == -INFINITY) ? 0.f : expf(s[r] - m_new);
                psum += p;
                if (p != 0.f) {                            // hidden keys hold whatever was there before
                    float vv[E];
                    Vec16d<ET>::load(vc + (size_t)(r * KPR + kir) * DH + part * E, vv);
#pragma unroll
                    for (int j = 0; j < E; ++j) acc[j] = fmaf(p, vv[j], acc[j]);
                }
            }
#pragma unroll
            for (int o = PARTS; o < 32; o <<= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
            l = l * corr + psum;
            m = m_new;
        }
        if (gave_up) s_bad = 1;
        parity ^= 1;
        __syncthreads();                           // everyone is done with the buffers before they are refilled
        if (s_bad) break;
    }
    if (gave_up && lane == 0) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);

    float* mine = wpart + warp * (DH + 2);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
    // lanes with the same piece hold sums over different keys: add them up
#pragma unroll
    for (int o = PARTS; o < 32; o <<= 1)
#pragma unroll
        for (int j = 0; j < E; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], o);
    if (lane < PARTS) {
#pragma unroll
        for (int j = 0; j < E; ++j) mine[2 + part * E + j] = acc[j];
    }
    __syncthreads();
    if (CLUSTER) finish_cluster<ET>(wpart, cpart, DH, row, h, split, n_split, out, ld_out);
    else finish_cta<ET>(wpart, DH, row, h, H, split, n_split, partials, counters, out, ld_out, &s_last);
}

template <typename ET, int DH>
int launch_bulk(dim3 grid, const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, const int* block_table,
                int max_blocks, const int* tok_slot, const int* tok_pos, void* out, int ld_out, int H, int Hkv, int BT,
                float scale, int window, int n_split, float* partials, int* counters, int* dev_err,
                cudaStream_t stream) {
    constexpr int CHUNK_BYTES = 32 * DH * (int)sizeof(ET);
    constexpr int CH_MAX = DEC_STAGE_BYTES / (2 * CHUNK_BYTES) < 8 ? DEC_STAGE_BYTES / (2 * CHUNK_BYTES) : 8;
    const size_t smem = 128 + (size_t)2 * CH_MAX * CHUNK_BYTES + (size_t)(DEC_WARPS + 1) * (DH + 2) * sizeof(float);
    // without scratch from the caller, the parts of a (row, head) merge inside a cluster (at most 16 CTAs)
    const bool cluster = n_split > 1 && n_split <= DEC_MAX_CLUSTER && partials == nullptr;
    auto kern = cluster ? attn_decode_bulk_kernel<ET, DH, true> : attn_decode_bulk_kernel<ET, DH, false>;
    static bool raised[2] = {false, false};
    if (!raised[cluster]) {
        cudaError_t e = cudaSuccess;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess && cluster) e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode: %zu bytes of shared memory, clusters: %s", smem, cudaGetErrorString(e));
        raised[cluster] = true;
    }
    cudaError_t e;
    if (cluster)
        e = launch_chained_cluster(kern, grid, dim3(DEC_WARPS * 32), smem, dim3(1, 1, n_split), stream, (const ET*)qkv, ld, q_off,
                                   (const ET*)Kc, (const ET*)Vc, block_table, max_blocks, tok_slot, tok_pos, (ET*)out,
                                   ld_out, H, Hkv, BT, scale, window, n_split, partials, counters, dev_err);
    else
        e = launch_chained(kern, grid, dim3(DEC_WARPS * 32), smem, stream, (const ET*)qkv, ld, q_off,
                           (const ET*)Kc, (const ET*)Vc, block_table, max_blocks, tok_slot, tok_pos, (ET*)out,
                           ld_out, H, Hkv, BT, scale, window, n_split, partials, counters, dev_err);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode: %s", cudaGetErrorString(e));
    return vlrf_check_launch("attn_decode");
}
// ---------------------------------------------------------------------------------------------------------
// bfloat16, head size 64: the same split-context attention with the two products on the tensor cores.
// A chunk of 32 keys (and values) arrives by a tiled TMA load with the 128-byte swizzle, so that `ldmatrix`
// reads it without bank conflicts.  A warp takes a chunk: S = q·Kᵀ as `mma.sync.m16n8k16` with the query in
// row 0 of the 16-row operand (the other rows are zeros), the softmax on the four lanes that hold row 0, P
// packed to bfloat16 straight from the accumulator registers, O += P·V with V read through transposing
// `ldmatrix`.  About a fifth of the instructions of the FMA kernel above, which stays for float32 and other
// head sizes.  Prefetch before the wait, merge of the warps and of the parts: as above.
__device__ __forceinline__ void dldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void dmma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t dpack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// address of the 16-byte piece `piece` (0…7) of row `row` of a [32][128 B] tile written with the 128-byte swizzle
__device__ __forceinline__ uint32_t dtile_addr(uint32_t base, int row, int piece) {
    return base + row * 128 + ((piece ^ (row & 7)) << 4);
}

template <bool CLUSTER>
__global__ void __launch_bounds__(DEC_WARPS * 32)
attn_decode_mma_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                       const __nv_bfloat16* __restrict__ qkv, int ld, int q_off, const int* __restrict__ block_table,
                       int max_blocks, const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                       __nv_bfloat16* __restrict__ out, int ld_out, int H, int Hkv, int BT, float scale, int window,
                       int n_split, float* __restrict__ partials, int* __restrict__ counters, int* __restrict__ dev_err,
                       long long* trace) {
    constexpr int DH = 64, CHUNK_BYTES = 32 * DH * 2, CH_MAX = 8;
    // (stations of the time stamps, kind 2: 0 the CTA begins, 1 the kernel ahead has finished, 2 warp 0's first chunk
    // is here, 3 warp 0 has worked through its chunks, 4 all warps have, 6 the merge is sent or, part 0, the row stored)
    const int tcta = (blockIdx.x * gridDim.y + blockIdx.y) * gridDim.z + blockIdx.z;
    if (threadIdx.x == 0) VLRF_TRACE(trace, 2, tcta, 0);
    extern __shared__ unsigned char dsm_raw[];
    unsigned char* dsm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(dsm_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* kbuf = dsm;                                                // [CH_MAX][32][128 B]
    unsigned char* vbuf = kbuf + (size_t)CH_MAX * CHUNK_BYTES;
    float* wpart = reinterpret_cast<float*>(vbuf + (size_t)CH_MAX * CHUNK_BYTES);   // [DEC_WARPS][DH + 2]
    float* crecv = wpart + DEC_WARPS * (DH + 2);                              // [DEC_MAX_CLUSTER][DH + 2] (CLUSTER, the CTA of part 0)
    uint64_t* bars = reinterpret_cast<uint64_t*>(crecv + DEC_MAX_CLUSTER * (DH + 2));   // CH_MAX barriers and the one of the merge
    uint64_t* cbar = bars + CH_MAX;
    __shared__ int s_last;
    static_assert(CH_MAX == DEC_WARPS, "a buffer and a barrier for every warp");
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
    if (threadIdx.x == 0) { tma_prefetch_descriptor(&tmap_k); tma_prefetch_descriptor(&tmap_v); }   // under the table reads
    // before the wait: positions, tables and the cache of earlier positions (see the kernel above)
    const int slot = tok_slot[row];
    if (slot < 0) return;                          // padding row: the whole CTA (and its cluster) leaves
    const int pos = tok_pos[row];
    const int hk = h / (H / Hkv);
    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    const int chunk0 = first / 32;
    const int n_chunks = pos / 32 + 1 - chunk0;
    const int per_split = (n_chunks + n_split - 1) / n_split;
    const int c_begin = chunk0 + split * per_split;
    const int c_end = min(chunk0 + n_chunks, c_begin + per_split);
    const int c_new = pos / 32;                    // the chunk with the key that the kernel ahead writes
    const int* table = block_table + (size_t)slot * max_blocks;

    if (threadIdx.x == 0) {
        for (int i = 0; i < CH_MAX; ++i) dmbar_init(&bars[i], 1);
        if (CLUSTER) dmbar_init(cbar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (CLUSTER && split == 0) dmbar_expect_tx(cbar, (uint32_t)(n_split * (DH + 2) * sizeof(float)));
    }
    __syncthreads();
    if (CLUSTER) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");   // (waited for before anyone sends)
    // Warp w streams the chunks c_begin + w, + 8, + 16, … through buffer w on barrier w, on its own: it asks for
    // its next chunk as soon as it has read the one before, and waits for no other warp until the merge.
    unsigned char* my_k = kbuf + (size_t)warp * CHUNK_BYTES;
    unsigned char* my_v = vbuf + (size_t)warp * CHUNK_BYTES;
    uint64_t* my_bar = &bars[warp];
    auto request = [&](int c, int blk) -> bool {   // one lane: chunk c, which lies in cache block blk, into this warp's buffer
        if (blk < 0) {
            atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
            return false;
        }
        const int k0 = c * 32;
        const int y = (blk * Hkv + hk) * BT + (k0 % BT);
        dmbar_expect_tx(my_bar, 2 * CHUNK_BYTES);
        tma_load_2d(my_k, &tmap_k, 0, y, my_bar);
        tma_load_2d(my_v, &tmap_v, 0, y, my_bar);
        return true;
    };
    const int my_first = c_begin + warp;
    int ok_first = 1;
    if (lane == 0 && my_first < c_end && my_first != c_new) ok_first = request(my_first, table[my_first * 32 / BT]) ? 1 : 0;
    if (CLUSTER) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    pdl_wait();                                    // the new key and value and the query are written
    if (threadIdx.x == 0) VLRF_TRACE(trace, 2, tcta, 1);
    pdl_launch_dependents();
    // the query as rows 0 of the MMA's 16-row operand: only lanes 0-3 hold anything but zeros
    uint32_t qa[4][2];
    {
        const __nv_bfloat16* qsrc = qkv + (size_t)row * ld + q_off + (size_t)h * DH;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            qa[ks][0] = g == 0 ? *reinterpret_cast<const uint32_t*>(qsrc + 16 * ks + 2 * t) : 0u;
            qa[ks][1] = g == 0 ? *reinterpret_cast<const uint32_t*>(qsrc + 16 * ks + 8 + 2 * t) : 0u;
        }
    }
    const float sl2 = scale * 1.4426950408889634f;       // scores in units of log2(e)

    float o[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f; }
    float m = -INFINITY, l = 0.f;
    bool gave_up = false, bad = false;
    uint32_t parity = 0;
    if (lane == 0 && my_first < c_end && my_first == c_new) ok_first = request(my_first, table[my_first * 32 / BT]) ? 1 : 0;
    if (!__shfl_sync(0xffffffffu, ok_first, 0)) bad = true;           // nothing of this warp's is in flight
    {
        for (int c = my_first; c < c_end && !bad; c += DEC_WARPS) {
            // the table entry of the chunk after this one, looked up while this one is on its way
            const int c_next = c + DEC_WARPS;
            int blk_next = 0;
            if (lane == 0 && c_next < c_end) blk_next = table[c_next * 32 / BT];
            uint32_t polls = 0;
            while (!dmbar_try_wait(my_bar, parity)) {
                if (++polls > DEC_WAIT_LIMIT) { gave_up = true; break; }
            }
            if (gave_up) break;
            if (threadIdx.x == 0 && c == my_first) VLRF_TRACE(trace, 2, tcta, 2);
            const int i = warp;
            const int k0 = c * 32;
            const uint32_t kb = dsmem_u32(kbuf + (size_t)i * CHUNK_BYTES), vb = dsmem_u32(vbuf + (size_t)i * CHUNK_BYTES);
            // Rows of the chunk behind the newest key hold whatever was there before; their scores are masked by
            // assignment below, but 0 · V would let a stray NaN through the MMA: clear those rows of V.
            const int valid = pos - k0 + 1;        // keys of this chunk that exist (at least 1)
            if (valid < 32) {
                unsigned char* vt = vbuf + (size_t)i * CHUNK_BYTES;
                for (int idx = lane; idx < (32 - valid) * 8; idx += 32)
                    *reinterpret_cast<uint4*>(vt + (valid + (idx >> 3)) * 128 + ((idx & 7) << 4)) = make_uint4(0, 0, 0, 0);
                __syncwarp();
            }
            float s[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
            for (int ks = 0; ks < 4; ks += 2) {
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    // matrices: (keys 8nt…, dims of k-step ks: low, high half), (same keys, k-step ks+1: low, high half)
                    uint32_t b0, b1, b2, b3;
                    dldsm_x4(dtile_addr(kb, nt * 8 + (lane & 7), ks * 2 + (lane >> 3)), b0, b1, b2, b3);
                    dmma16816(s[nt], qa[ks][0], 0u, qa[ks][1], 0u, b0, b1);
                    dmma16816(s[nt], qa[ks + 1][0], 0u, qa[ks + 1][1], 0u, b2, b3);
                }
            }
            // row 0 of S lies in lanes 0-3: keys k0 + 8nt + 2t and + 1; the other lanes hold rows of zeros
            float cmax = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = k0 + nt * 8 + 2 * t + e;
                    const float v = (g == 0 && key >= first && key <= pos) ? s[nt][e] * sl2 : -INFINITY;
                    s[nt][e] = v;
                    cmax = fmaxf(cmax, v);
                }
            cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 1));
            cmax = fmaxf(cmax, __shfl_xor_sync(0xffffffffu, cmax, 2));
            const float m_new = fmaxf(m, cmax);
            const float m_use = (m_new == -INFINITY) ? 0.f : m_new;      // (lanes beside row 0: every p is 0)
            const float corr = (m == -INFINITY) ? 0.f : exp2f(m - m_new);
            float psum = 0.f;
            uint32_t pa[4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                const float p0 = exp2f(s[nt][0] - m_use), p1 = exp2f(s[nt][1] - m_use);
                psum += p0 + p1;
                pa[nt] = dpack_bf16(p0, p1);
            }
            psum += __shfl_xor_sync(0xffffffffu, psum, 1);
            psum += __shfl_xor_sync(0xffffffffu, psum, 2);
            l = l * corr + psum;
            m = m_new;
#pragma unroll
            for (int j = 0; j < 8; ++j) { o[j][0] *= corr; o[j][1] *= corr; }
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
                for (int j = 0; j < 8; j += 2) {
                    // transposed loads: (keys 16kk…+7, dims 8j…), (keys +8…, same dims), then the same for dims 8(j+1)…
                    uint32_t b0, b1, b2, b3;
                    dldsm_x4_trans(dtile_addr(vb, kk * 16 + (lane & 15), j + (lane >> 4)), b0, b1, b2, b3);
                    dmma16816(o[j], pa[2 * kk], 0u, pa[2 * kk + 1], 0u, b0, b1);
                    dmma16816(o[j + 1], pa[2 * kk], 0u, pa[2 * kk + 1], 0u, b2, b3);
                }
            }
            parity ^= 1;
            if (c_next < c_end) {
                // the warp's reads of its buffer (and the rows of V it cleared) come before the copy that refills it
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                int ok_next = 1;
                if (lane == 0) ok_next = request(c_next, blk_next) ? 1 : 0;
                if (!__shfl_sync(0xffffffffu, ok_next, 0)) bad = true;      // (the loop ends with nothing in flight)
            }
        }
    }
    if (gave_up && lane == 0) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
    if (threadIdx.x == 0) VLRF_TRACE(trace, 2, tcta, 3);

    // this warp's (maximum, sum, outputs): row 0 lies in lanes 0-3, dimensions 8j + 2t and + 1; the merge
    // works with natural logarithms
    float* mine = wpart + warp * (DH + 2);
    if (lane == 0) { mine[0] = m * 0.6931471805599453f; mine[1] = l; }
    if (g == 0) {
#pragma unroll
        for (int j = 0; j < 8; ++j) { mine[2 + 8 * j + 2 * t] = o[j][0]; mine[2 + 8 * j + 2 * t + 1] = o[j][1]; }
    }
    __syncthreads();
    if (threadIdx.x == 0) VLRF_TRACE(trace, 2, tcta, 4);
    if (CLUSTER) finish_cluster_push<__nv_bfloat16, DH>(wpart, crecv, cbar, row, h, split, n_split, out, ld_out, dev_err);
    else finish_cta<__nv_bfloat16>(wpart, DH, row, h, H, split, n_split, partials, counters, out, ld_out, &s_last);
    if (threadIdx.x == 0) VLRF_TRACE(trace, 2, tcta, 6);
}

int launch_mma(dim3 grid, const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, long long kv_rows,
               const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos, void* out, int ld_out,
               int H, int Hkv, int BT, float scale, int window, int n_split, float* partials, int* counters,
               int* dev_err, cudaStream_t stream) {
    CUtensorMap tk, tv;
    int st = vlrf_make_tmap_bf16(Kc, kv_rows, 64, 64, 32, 64, &tk);
    if (st != VLRF_OK) return st;
    st = vlrf_make_tmap_bf16(Vc, kv_rows, 64, 64, 32, 64, &tv);
    if (st != VLRF_OK) return st;
    const size_t smem = 1024 + (size_t)2 * 8 * 4096 + (size_t)(DEC_WARPS + DEC_MAX_CLUSTER) * (64 + 2) * sizeof(float) + 9 * 8;
    const bool cluster = n_split > 1 && n_split <= DEC_MAX_CLUSTER && partials == nullptr;
    auto kern = cluster ? attn_decode_mma_kernel<true> : attn_decode_mma_kernel<false>;
    static bool raised[2] = {false, false};
    if (!raised[cluster]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess && cluster) e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode: %zu bytes of shared memory, clusters: %s", smem, cudaGetErrorString(e));
        raised[cluster] = true;
    }
    cudaError_t e;
    if (cluster)
        e = launch_chained_cluster(kern, grid, dim3(DEC_WARPS * 32), smem, dim3(1, 1, n_split), stream, tk, tv,
                                   (const __nv_bfloat16*)qkv, ld, q_off, block_table, max_blocks, tok_slot, tok_pos,
                                   (__nv_bfloat16*)out, ld_out, H, Hkv, BT, scale, window, n_split, partials, counters, dev_err,
                                   vlrf_trace_buffer());
    else
        e = launch_chained(kern, grid, dim3(DEC_WARPS * 32), smem, stream, tk, tv, (const __nv_bfloat16*)qkv, ld, q_off,
                           block_table, max_blocks, tok_slot, tok_pos, (__nv_bfloat16*)out, ld_out, H, Hkv, BT, scale,
                           window, n_split, partials, counters, dev_err, vlrf_trace_buffer());
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode: %s", cudaGetErrorString(e));
    return vlrf_check_launch("attn_decode");
}
}  // namespace

// Whether a context cut into n_split parts needs scratch from the caller (else the parts' CTAs form a
// cluster and merge through shared memory).
extern "C" int vlrf_attn_decode_needs_scratch(int dh, int n_split) {
    return (n_split > 1 && !((dh == 64 || dh == 128) && n_split <= DEC_MAX_CLUSTER)) ? 1 : 0;
}

// floats of scratch for the partials and ints for the counters
extern "C" long long vlrf_attn_decode_scratch_floats(int rows, int H, int dh, int n_split) {
    return (long long)rows * H * n_split * (dh + 2);
}

// n_blocks: blocks of the cache (for the tensor-core kernel's tensor maps), or 0 if the caller does not say
static int attn_decode_impl(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                            const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos,
                            void* out, int ld_out, int rows, int H, int Hkv, int dh, int BT, float scale,
                            int window, int n_split, float* partials, int* counters, int* dev_err,
                            cudaStream_t stream) {
    VLRF_REQUIRE(rows >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "attn_decode: bad sizes");
    VLRF_REQUIRE(H % Hkv == 0, "attn_decode: %d heads cannot share %d key/value heads", H, Hkv);
    VLRF_REQUIRE(dh > 0 && dh % 16 == 0 && dh <= DEC_MAX_DH,
                 "attn_decode: head size %d is not a multiple of 16 up to %d", dh, DEC_MAX_DH);
    VLRF_REQUIRE(BT % 32 == 0, "attn_decode: cache blocks of %d tokens are not a multiple of 32", BT);
    VLRF_REQUIRE(n_split >= 1 && n_split <= 65535 && H <= 65535, "attn_decode: bad split %d", n_split);
    const bool clustered = (dh == 64 || dh == 128) && n_split <= DEC_MAX_CLUSTER;    // merges in shared memory
    VLRF_REQUIRE(n_split == 1 || clustered || (partials != nullptr && counters != nullptr),
                 "attn_decode: this split context needs scratch");
    if (partials == nullptr || counters == nullptr) partials = nullptr, counters = nullptr;
    VLRF_REQUIRE(window >= 0 && dev_err != nullptr, "attn_decode: bad window or no error word");
    if (rows == 0) return VLRF_OK;
    dim3 grid(rows, H, n_split);
    if (dtype == VLRF_BF16 && dh == 64 && n_blocks > 0 && ld % 2 == 0 && q_off % 2 == 0)
        return launch_mma(grid, qkv, ld, q_off, Kc, Vc, (long long)n_blocks * Hkv * BT, block_table, max_blocks, tok_slot, tok_pos,
                          out, ld_out, H, Hkv, BT, scale, window, n_split, partials, counters, dev_err, stream);
#define BULK(ET, DHT) return launch_bulk<ET, DHT>(grid, qkv, ld, q_off, Kc, Vc, block_table, max_blocks, tok_slot, tok_pos, \
                                                  out, ld_out, H, Hkv, BT, scale, window, n_split, partials, counters, dev_err, stream)
    if (dtype == VLRF_BF16 && dh == 64) BULK(__nv_bfloat16, 64);
    if (dtype == VLRF_BF16 && dh == 128) BULK(__nv_bfloat16, 128);
    if (dtype == VLRF_F32 && dh == 64) BULK(float, 64);
    if (dtype == VLRF_F32 && dh == 128) BULK(float, 128);
#undef BULK
    const size_t smem = (size_t)(dh + DEC_WARPS * (dh + 2)) * sizeof(float);
    if (dtype == VLRF_F32)
        attn_decode_generic_kernel<float><<<grid, DEC_WARPS * 32, smem, stream>>>(
            (const float*)qkv, ld, q_off, (const float*)Kc, (const float*)Vc, block_table, max_blocks, tok_slot,
            tok_pos, (float*)out, ld_out, H, Hkv, dh, BT, scale, window, n_split, partials, counters, dev_err);
    else if (dtype == VLRF_BF16)
        attn_decode_generic_kernel<__nv_bfloat16><<<grid, DEC_WARPS * 32, smem, stream>>>(
            (const __nv_bfloat16*)qkv, ld, q_off, (const __nv_bfloat16*)Kc, (const __nv_bfloat16*)Vc, block_table,
            max_blocks, tok_slot, tok_pos, (__nv_bfloat16*)out, ld_out, H, Hkv, dh, BT, scale, window, n_split,
            partials, counters, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "attn_decode: unknown dtype %d", dtype);
    return vlrf_check_launch("attn_decode");
}

extern "C" int vlrf_attn_decode(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc,
                                int n_blocks, const int* block_table, int max_blocks, const int* tok_slot,
                                const int* tok_pos, void* out, int ld_out, int rows, int H, int Hkv, int dh,
                                int BT, float scale, int window, int n_split, float* partials, int* counters,
                                int* dev_err, cudaStream_t stream) {
    return attn_decode_impl(qkv, dtype, ld, q_off, Kc, Vc, n_blocks, block_table, max_blocks, tok_slot, tok_pos, out, ld_out,
                            rows, H, Hkv, dh, BT, scale, window, n_split, partials, counters, dev_err, stream);
}

// ---------------------------------------------------------------------------------------------------------
// The same decode attention for callers that must not allocate (declared in attention_decode_noalloc.h).
// Its scratch memory lives in this library's image instead of coming from the caller.
#include "attention_decode_noalloc.h"
#include <mutex>

static __device__ __align__(256) float g_noalloc_partials[VLRF_NOALLOC_MAX_PARTIAL_FLOATS];
static __device__ __align__(256) int g_noalloc_counters[VLRF_NOALLOC_MAX_ROW_HEADS];

namespace {
constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_partials_addr[NOALLOC_MAX_DEVICES] = {nullptr};
int* g_noalloc_counters_addr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace

extern "C" int vlrf_attn_decode_noalloc(const void* qkv, int dtype, int ld, int q_off, const void* Kc,
                                        const void* Vc, const int* block_table, int max_blocks,
                                        const int* tok_slot, const int* tok_pos, void* out, int ld_out,
                                        int rows, int H, int Hkv, int dh, int BT, float scale, int window,
                                        int n_split, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(rows >= 0 && H > 0 && n_split >= 1 && dh > 0, "attn_decode_noalloc: bad sizes");
    VLRF_REQUIRE((long long)rows * H <= VLRF_NOALLOC_MAX_ROW_HEADS,
                 "attn_decode_noalloc: %d rows x %d heads exceed the built-in scratch for %d (row, head) pairs",
                 rows, H, VLRF_NOALLOC_MAX_ROW_HEADS);
    VLRF_REQUIRE((long long)rows * H * n_split * (dh + 2) <= VLRF_NOALLOC_MAX_PARTIAL_FLOATS,
                 "attn_decode_noalloc: %d rows x %d heads x %d splits x head size %d exceed the built-in scratch of %d floats",
                 rows, H, n_split, dh, VLRF_NOALLOC_MAX_PARTIAL_FLOATS);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
    VLRF_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, "attn_decode_noalloc: device %d is beyond the %d this entry point tracks", dev, NOALLOC_MAX_DEVICES);
    float* partials = nullptr;
    int* counters = nullptr;
    {
        // Set-up, once per device, with that device current: in host code the arrays' names are only
        // stand-ins; their device addresses have to be asked for.
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (g_noalloc_partials_addr[dev] == nullptr) {
            float* p = nullptr;
            int* c = nullptr;
            e = cudaGetSymbolAddress((void**)&p, g_noalloc_partials);
            if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode_noalloc: address of the partials: %s", cudaGetErrorString(e));
            e = cudaGetSymbolAddress((void**)&c, g_noalloc_counters);
            if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode_noalloc: address of the counters: %s", cudaGetErrorString(e));
            g_noalloc_partials_addr[dev] = p;
            g_noalloc_counters_addr[dev] = c;
        }
        partials = g_noalloc_partials_addr[dev];
        counters = g_noalloc_counters_addr[dev];
    }
    if (n_split > 1 && rows > 0) {
        // the counters must start at zero; whatever an earlier call left is cleared (no allocation involved)
        e = cudaMemsetAsync(counters, 0, (size_t)rows * H * sizeof(int), stream);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "attn_decode_noalloc: clearing the counters: %s", cudaGetErrorString(e));
    }
    return attn_decode_impl(qkv, dtype, ld, q_off, Kc, Vc, 0, block_table, max_blocks, tok_slot, tok_pos, out, ld_out,
                            rows, H, Hkv, dh, BT, scale, window, n_split, partials, counters, dev_err, stream);
}
