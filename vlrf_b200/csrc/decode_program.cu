// A whole decode step as ONE persistent kernel that runs a list of operations.
//
// A decode step of a small batch is a chain of some sixty tiny dependent operations (norm + projection,
// attention, projection + residual, ...).  As sixty launches each pays its own start-up, and none streams
// long enough to come near the memory rate.  Here one CTA per SM stays resident for the whole step and all CTAs
// walk the same list of operations; between two operations they meet at a barrier over the grid (a counter
// in global memory, bounded polling).  What the list holds is decided by the model's parts on the host:
// this file knows three kinds of operation and no architecture.
//
//   EMBED      x[r] = wte[token[r]] + wpe[position[r]]                           float32 rows
//   GEMV       out[r] = act(norm(in[r]) · Wᵀ + bias) (+ residual[r])             few rows, W [N][K] bfloat16
//              norm: none, LayerNorm (two passes, float32) or RMS norm, applied while the rows are staged;
//              optionally the K and V columns of the result are also written into a paged cache
//   ATTENTION  one query per (row, head) over the keys 0…position of its slot in a paged cache,
//              float32 online softmax, the context cut into parts that the last CTA to finish merges in order
//
// Weights never depend on an earlier operation, so one warp of each CTA (the producer) streams this CTA's share
// of every operation's weights through a ring of shared-memory slots with bulk copies, as far ahead as
// the ring allows, across operation boundaries; HBM stays busy while the other eight warps wait at barriers.
// The products run on `mma.sync` (bfloat16 in, float32 accumulate) with the rows as the 16-row operand; a 16-byte
// shared-memory read feeds two MMAs through a permutation of k that both operands share.  A unit of work of a
// GEMV is 8 or 16 output columns over one chunk of k; the eight warps split the chunk's 32-wide pieces and add
// their partial tiles through shared memory in a fixed order, so results do not depend on timing.
//
// All CTAs must be resident at once: the kernel is launched cooperatively with one CTA per SM.  Every wait (grid
// barrier, ring slot) is bounded; a wait that runs out sets VLRF_DEVERR_WAIT_TIMEOUT and a flag that makes every
// CTA leave the kernel.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int DP_CONSUMER_WARPS = 8;
constexpr int DP_CONSUMERS = 32 * DP_CONSUMER_WARPS;
constexpr int DP_THREADS = DP_CONSUMERS + 32;
constexpr int DP_MAX_ROWS = 16;
constexpr int DP_SLOT_BYTES = 32 * 1024;
constexpr int DP_SLOTS = 5;
constexpr int DP_STAGE_BYTES = 52 * 1024;
constexpr int DP_RED_FLOATS = DP_CONSUMER_WARPS * 16 * 16;
constexpr int DP_TABLE_INTS = 1024;
constexpr int DP_MAX_K_SINGLE = 2016;               // a normed GEMV keeps a whole row in registers: 16 float4 a lane
constexpr uint32_t DP_GRID_WAIT_LIMIT = 1u << 22;   // polls of the grid counter before a wait gives up
constexpr int DP_ATT_UNROLL = 8;
constexpr int DP_BIAS_BYTES = 64;                   // room behind a slot's weight rows for the bias of its columns

enum { DP_EMBED = 0, DP_GEMV = 1, DP_ATTENTION = 2 };
enum { DP_NORM_NONE = 0, DP_NORM_LAYER = 1, DP_NORM_RMS = 2 };

struct alignas(16) DecodeOp {
    int32_t kind, N, K, in_f32, norm, act, out_f32, ld_out;
    float eps, scale;
    int32_t k_off, v_off, hkv, dh, bt, table_ld;
    int32_t n_heads, q_off, ld_in, n_split, window, vocab, n_pos, pad0;
    const void* in;
    const float* gamma;
    const float* beta;
    const void* W;
    const float* bias;
    void* out;
    const float* residual;
    void* kc;
    void* vc;
    const int* table;
    float* partials;
    int* counters;
    const void* wpe;
    const int* tokens;
};

// How a GEMV is cut: chunks of k (each a multiple of 32 that fits a ring slot at 8 columns and the staging area
// at `rows_pad` rows), and 16 output columns a unit where a slot holds them, else 8.
struct GemvPlan { int n_kchunks, kchunk, ncols, w_stride, a_stride; };

__host__ __device__ inline int dp_pad_stride(int bytes) {   // row stride ≡ 64 (mod 128): 16-byte reads of 8 rows hit 32 banks
    return bytes + ((64 - bytes % 128) + 128) % 128;
}
__host__ __device__ inline bool dp_plan_gemv(int n_rows, int K, GemvPlan* p) {
    if (K <= 0 || K % 32 != 0) return false;
    const int rows_pad = n_rows <= 8 ? 8 : 16;
    int limit = (DP_STAGE_BYTES / rows_pad - 128) / 2;
    const int slot_limit = ((DP_SLOT_BYTES - DP_BIAS_BYTES) / 8 - 128) / 2;
    if (slot_limit < limit) limit = slot_limit;
    limit -= limit % 32;
    int n = (K + limit - 1) / limit;
    while (K % (n * 32) != 0) ++n;
    p->n_kchunks = n;
    p->kchunk = K / n;
    p->w_stride = dp_pad_stride(p->kchunk * 2);
    p->a_stride = p->w_stride;
    p->ncols = 16 * p->w_stride + DP_BIAS_BYTES <= DP_SLOT_BYTES ? 16 : 8;
    return true;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DP_CONSUMERS) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int ld_volatile_i32(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint4 ldcg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float4 ldcg_f4(const void* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tsm(dst)), "l"(src), "r"(bytes), "r"(tsm(bar)) : "memory");
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

struct Shared {
    uint64_t full[DP_SLOTS];
    uint64_t empty[DP_SLOTS];
    int abort_flag;      // a wait ran out somewhere: every later wait is skipped, and the step ends at the next barrier
    int go_flag;         // what the grid barrier found, written by one thread between two CTA barriers
    int last_flag;
    int table_ld;
    const int* table_of;
    int tok_slot[DP_MAX_ROWS];
    int tok_pos[DP_MAX_ROWS];
    DecodeOp op[2];      // the operation being run and the next one, fetched while the CTA waits at the grid barrier
};

struct Ctx {
    Shared* sh;
    unsigned char* ring;
    unsigned char* stage;
    float* red;
    int* table;
    unsigned* sync_words;    // [0] barrier counter, [1] exit counter, [2] abort flag
    int* dev_err;
    long long* trace;        // or null: one CTA notes the time (ns) at which it begins every operation, and the end
    unsigned trace_cta;
    int n_rows;
    unsigned grid;
};

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// trace[op][k], k = 0: the operation begins; 1: its rows are staged; 2: its first weights have landed; 3: products
// done; 4: results stored; 5: arrived at the grid barrier.  Written by the first thread of the CTA that sync_words[3] names.
constexpr int DP_TRACE_STAMPS = 8;
__device__ __forceinline__ void stamp(const Ctx& c, int op_index, int k) {
    if (c.trace != nullptr && threadIdx.x == 0 && blockIdx.x == c.trace_cta) c.trace[op_index * DP_TRACE_STAMPS + k] = global_ns();
}

__device__ __forceinline__ void raise_abort(const Ctx& c) {
    c.sh->abort_flag = 1;
    atomicOr(c.dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
    atomicExch(reinterpret_cast<int*>(c.sync_words + 2), 1);
}

// All consumer threads of all CTAs: what every CTA wrote before is visible to every CTA after.  Returns false
// when the step is being abandoned.
//
// One thread of the CTA arrives with a release (the CTA barrier before it makes the other threads' writes part of
// what is released) and polls with acquire loads, two of them in flight so that the last arrival is seen about half
// a round trip to L2 earlier; the CTA barrier after it hands what was acquired to the other threads.
__device__ bool grid_barrier(const Ctx& c, unsigned target, const DecodeOp* next_op, DecodeOp* next_buf) {
    consumer_sync();
    if (next_op != nullptr && threadIdx.x >= 32 && threadIdx.x < 32 + (int)(sizeof(DecodeOp) / 4))
        reinterpret_cast<uint32_t*>(next_buf)[threadIdx.x - 32] = __ldg(reinterpret_cast<const uint32_t*>(next_op) + threadIdx.x - 32);
    stamp(c, (int)(target / c.grid) - 1, 4);
    if (threadIdx.x == 0) {
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(c.sync_words) : "memory");
        stamp(c, (int)(target / c.grid) - 1, 5);
        uint32_t polls = 0;
        unsigned v0 = ld_acquire_u32(c.sync_words);
        __nanosleep(200);
        for (;;) {
            const unsigned v1 = ld_acquire_u32(c.sync_words);     // asked for while v0 is still on its way
            if (v0 >= target) break;
            v0 = ld_acquire_u32(c.sync_words);
            if (v1 >= target) break;
            ++polls;
            if ((polls & 127u) == 0 && ld_volatile_i32(reinterpret_cast<const int*>(c.sync_words + 2))) {
                c.sh->abort_flag = 1;
                break;
            }
            if (polls > DP_GRID_WAIT_LIMIT) {
                raise_abort(c);
                break;
            }
        }
        c.sh->go_flag = c.sh->abort_flag == 0;
    }
    consumer_sync();
    return c.sh->go_flag != 0;
}

__device__ __forceinline__ int block_of(const Ctx& c, const DecodeOp& op, int row, int slot, int block_index) {
    if (c.sh->table_of == op.table) return c.table[row * c.sh->table_ld + block_index];
    return __ldg(op.table + (size_t)slot * op.table_ld + block_index);
}

// ---- the producer warp: this CTA's weight tiles of every operation, in the order the consumers use them ----
__device__ void produce(const Ctx& c, const DecodeOp* __restrict__ ops, int n_ops) {
    const int lane = threadIdx.x & 31;
    uint32_t filled = 0;
    for (int i = 0; i < n_ops; ++i) {
        const DecodeOp& op = ops[i];
        if (op.kind != DP_GEMV) continue;
        GemvPlan p;
        dp_plan_gemv(c.n_rows, op.K, &p);
        const int n_units = (op.N + p.ncols - 1) / p.ncols;
        const unsigned rot = (unsigned)(i * 53) % c.grid;
        const unsigned char* W = static_cast<const unsigned char*>(op.W);
        const unsigned first = (blockIdx.x + c.grid - rot) % c.grid;
        if (first < (unsigned)n_units && op.norm != DP_NORM_NONE) {
            // the norm's weight and bias, a slot of their own: [gamma K floats][beta K floats]
            const int slot = filled % DP_SLOTS;
            const uint32_t round = filled / DP_SLOTS;
            if (round > 0 && !tbar_wait_or_abort(&c.sh->empty[slot], (round - 1) & 1, &c.sh->abort_flag)) {
                if (lane == 0 && !c.sh->abort_flag) raise_abort(c);
                return;
            }
            unsigned char* dst = c.ring + (size_t)slot * DP_SLOT_BYTES;
            if (lane == 0) {
                tbar_expect_tx(&c.sh->full[slot], (uint32_t)op.K * 4 * (op.beta != nullptr ? 2 : 1));
                bulk_g2s(dst, op.gamma, (uint32_t)op.K * 4, &c.sh->full[slot]);
                if (op.beta != nullptr) bulk_g2s(dst + (size_t)op.K * 4, op.beta, (uint32_t)op.K * 4, &c.sh->full[slot]);
            }
            __syncwarp();
            ++filled;
        }
        for (unsigned u = first; u < (unsigned)n_units; u += c.grid) {
            const int n0 = u * p.ncols;
            const int rows = min(p.ncols, op.N - n0);
            const bool with_bias = op.bias != nullptr && rows % 4 == 0;
            for (int kc = 0; kc < p.n_kchunks; ++kc, ++filled) {
                const int slot = filled % DP_SLOTS;
                const uint32_t round = filled / DP_SLOTS;
                if (round > 0 && !tbar_wait_or_abort(&c.sh->empty[slot], (round - 1) & 1, &c.sh->abort_flag)) {
                    if (lane == 0 && !c.sh->abort_flag) raise_abort(c);
                    return;
                }
                unsigned char* dst = c.ring + (size_t)slot * DP_SLOT_BYTES;
                const bool bias_here = with_bias && kc == 0;
                if (lane == 0) tbar_expect_tx(&c.sh->full[slot], (uint32_t)rows * p.kchunk * 2 + (bias_here ? rows * 4 : 0));
                __syncwarp();
                if (lane < rows)
                    bulk_g2s(dst + (size_t)lane * p.w_stride, W + ((size_t)(n0 + lane) * op.K + (size_t)kc * p.kchunk) * 2,
                             (uint32_t)p.kchunk * 2, &c.sh->full[slot]);
                if (lane == 31 && bias_here)
                    bulk_g2s(dst + (size_t)p.ncols * p.w_stride, op.bias + n0, (uint32_t)rows * 4, &c.sh->full[slot]);
            }
        }
    }
}

// ---- staging the rows of a GEMV: norm in float32, result bfloat16 [rows][a_stride bytes] ----
// Every load of a row is asked for before the first is used (a loop of their own, addresses clamped instead of
// loads predicated): written the obvious way, each load was followed by its use and the round trips to L2 ran one
// after another.  NJ: float4 a lane.  (`params`: the norm's weight, then its bias, in shared memory)
template <int NJ>
__device__ void stage_normed_t(const Ctx& c, const DecodeOp& op, const GemvPlan& p, const float* params) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = op.K, nv = K / 4, norm = op.norm;
    const float eps = op.eps;
    const bool with_beta = op.beta != nullptr;
    const float* X = static_cast<const float*>(op.in);
    const int ld = op.ld_in;
    for (int r = warp; r < c.n_rows; r += DP_CONSUMER_WARPS) {
        const float* xr = X + (size_t)r * ld;
        float4 v[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) v[j] = ldcg_f4(xr + 4 * min(lane + 32 * j, nv - 1));
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            if (lane + 32 * j >= nv) v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        float mean = 0.f, rstd = 1.f;
        if (norm == DP_NORM_LAYER) {
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) sum += (v[j].x + v[j].y) + (v[j].z + v[j].w);
            mean = warp_sum(sum) / (float)K;
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                if (lane + 32 * j < nv) {
                    const float a = v[j].x - mean, b = v[j].y - mean, cc = v[j].z - mean, d = v[j].w - mean;
                    sq += (a * a + b * b) + (cc * cc + d * d);
                }
            }
            rstd = rsqrtf(warp_sum(sq) / (float)K + eps);
        } else if (norm == DP_NORM_RMS) {
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) sq += (v[j].x * v[j].x + v[j].y * v[j].y) + (v[j].z * v[j].z + v[j].w * v[j].w);
            rstd = rsqrtf(warp_sum(sq) / (float)K + eps);
        }
        unsigned char* row = c.stage + (size_t)r * p.a_stride;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int i = lane + 32 * j;
            if (i < nv) {
                float4 y = make_float4((v[j].x - mean) * rstd, (v[j].y - mean) * rstd, (v[j].z - mean) * rstd,
                                       (v[j].w - mean) * rstd);
                if (norm != DP_NORM_NONE) {
                    const float4 g = reinterpret_cast<const float4*>(params)[i];
                    y.x *= g.x; y.y *= g.y; y.z *= g.z; y.w *= g.w;
                    if (with_beta) {
                        const float4 b = reinterpret_cast<const float4*>(params + K)[i];
                        y.x += b.x; y.y += b.y; y.z += b.z; y.w += b.w;
                    }
                }
                uint2 o;
                o.x = pack2(y.x, y.y);
                o.y = pack2(y.z, y.w);
                *reinterpret_cast<uint2*>(row + 8 * i) = o;
            }
        }
    }
}
__device__ void stage_normed(const Ctx& c, const DecodeOp& op, const GemvPlan& p, const float* params) {
    const int nj = (op.K / 4 + 31) / 32;
    if (nj <= 2) stage_normed_t<2>(c, op, p, params);
    else if (nj <= 4) stage_normed_t<4>(c, op, p, params);
    else if (nj <= 6) stage_normed_t<6>(c, op, p, params);
    else if (nj <= 8) stage_normed_t<8>(c, op, p, params);
    else if (nj <= 10) stage_normed_t<10>(c, op, p, params);
    else if (nj <= 13) stage_normed_t<13>(c, op, p, params);
    else stage_normed_t<16>(c, op, p, params);
}

__device__ __forceinline__ void cp_async_16(void* dst_shared, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tsm(dst_shared)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}

// bfloat16 rows (or float32 rows of a width that is staged in chunks): columns [k0, k0 + kchunk).  bfloat16 rows
// are copied asynchronously, all pieces in flight at once.
__device__ void stage_plain(const Ctx& c, const DecodeOp& op, const GemvPlan& p, int k0) {
    const int tid = threadIdx.x;
    const int pieces = p.kchunk / 8;                    // 16-byte pieces a row
    const int ld = op.ld_in;
    if (!op.in_f32) {
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(op.in) + k0;
        for (int i = tid; i < c.n_rows * pieces; i += DP_CONSUMERS) {
            const int r = i / pieces, q = i % pieces;
            cp_async_16(c.stage + (size_t)r * p.a_stride + 16 * q, src + (size_t)r * ld + 8 * q);
        }
        cp_async_wait_all();
        return;
    }
    for (int i = tid; i < c.n_rows * pieces; i += DP_CONSUMERS) {
        const int r = i / pieces, q = i % pieces;
        const float* src = static_cast<const float*>(op.in) + (size_t)r * ld + k0 + 8 * q;
        const float4 a = ldcg_f4(src), b = ldcg_f4(src + 4);
        *reinterpret_cast<uint4*>(c.stage + (size_t)r * p.a_stride + 16 * q) =
            make_uint4(pack2(a.x, a.y), pack2(a.z, a.w), pack2(b.x, b.y), pack2(b.z, b.w));
    }
}

// `slot_bias`: the bias of the unit's columns in shared memory, or null (then it is read from global memory);
// `residual_value`: the residual of this thread's element if it was fetched ahead (have_residual)
__device__ void gemv_epilogue(const Ctx& c, const DecodeOp& op, const GemvPlan& p, int n0, const float* slot_bias,
                              bool have_residual, float residual_value) {
    const int tid = threadIdx.x;
    const int r = tid / p.ncols, cn = tid % p.ncols;
    const int n = n0 + cn;
    if (tid >= 16 * p.ncols || r >= c.n_rows || n >= op.N) return;
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < DP_CONSUMER_WARPS; ++w) v += c.red[(w * 16 + r) * 16 + cn];
    if (op.bias != nullptr) v += slot_bias != nullptr ? slot_bias[cn] : __ldg(op.bias + n);
    if (op.act == VLRF_ACT_GELU_TANH) v = op.out_f32 ? gelu_tanh_f(v) : gelu_tanh_fast(v);
    else if (op.act == VLRF_ACT_GELU_ERF) v = gelu_erf_f(v);
    if (op.residual != nullptr) v += have_residual ? residual_value : __ldcg(op.residual + (size_t)r * op.ld_out + n);
    if (op.out_f32) {
        static_cast<float*>(op.out)[(size_t)r * op.ld_out + n] = v;
        return;
    }
    const __nv_bfloat16 o = __float2bfloat16_rn(v);
    static_cast<__nv_bfloat16*>(op.out)[(size_t)r * op.ld_out + n] = o;
    if (op.kc == nullptr) return;
    const int width = op.hkv * op.dh;
    __nv_bfloat16* cache = nullptr;
    int col = 0;
    if (n >= op.k_off && n < op.k_off + width) { cache = static_cast<__nv_bfloat16*>(op.kc); col = n - op.k_off; }
    else if (n >= op.v_off && n < op.v_off + width) { cache = static_cast<__nv_bfloat16*>(op.vc); col = n - op.v_off; }
    if (cache == nullptr) return;
    const int slot = c.sh->tok_slot[r], pos = c.sh->tok_pos[r];
    if (slot < 0) return;
    const int blk = block_of(c, op, r, slot, pos / op.bt);
    if (blk < 0) { atomicOr(c.dev_err, VLRF_DEVERR_NO_BLOCK); return; }
    cache[(((size_t)blk * op.hkv + col / op.dh) * op.bt + pos % op.bt) * op.dh + col % op.dh] = o;
}

// No thread leaves an operation early: a wait that runs out raises the abort flag and the thread goes on (with
// meaningless numbers) to the next barrier of its CTA, so that the CTA's barriers always see all their threads.
__device__ void run_gemv(const Ctx& c, const DecodeOp& op, int op_index, uint32_t& consumed) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    GemvPlan p;
    dp_plan_gemv(c.n_rows, op.K, &p);
    const int n_units = (op.N + p.ncols - 1) / p.ncols;
    const unsigned rot = (unsigned)(op_index * 53) % c.grid;
    const unsigned first = (blockIdx.x + c.grid - rot) % c.grid;
    if (first >= (unsigned)n_units) return;
    const bool high_rows = c.n_rows > 8;
    const int n_pieces = p.kchunk / 32;
    const bool normed = op.norm != DP_NORM_NONE || (op.in_f32 && p.n_kchunks == 1 && op.K <= DP_MAX_K_SINGLE);
    // the residual of this thread's element of the first unit: asked for now, used in the epilogue
    float residual_first = 0.f;
    if (op.residual != nullptr) {
        const int r = threadIdx.x / p.ncols, n = first * p.ncols + threadIdx.x % p.ncols;
        if (threadIdx.x < 16 * p.ncols && r < c.n_rows && n < op.N) residual_first = __ldcg(op.residual + (size_t)r * op.ld_out + n);
    }
    stamp(c, op_index, 6);
    const float* params = nullptr;
    int param_slot = -1;
    if (op.norm != DP_NORM_NONE) {
        param_slot = consumed % DP_SLOTS;
        if (!c.sh->abort_flag && !tbar_wait_or_abort(&c.sh->full[param_slot], (consumed / DP_SLOTS) & 1, &c.sh->abort_flag) &&
            lane == 0 && !c.sh->abort_flag)
            raise_abort(c);
        params = reinterpret_cast<const float*>(c.ring + (size_t)param_slot * DP_SLOT_BYTES);
        ++consumed;
    }
    stamp(c, op_index, 7);
    if (p.n_kchunks == 1) {
        if (normed) stage_normed(c, op, p, params); else stage_plain(c, op, p, 0);
        consumer_sync();
    }
    if (param_slot >= 0 && lane == 0) tbar_arrive(&c.sh->empty[param_slot]);
    stamp(c, op_index, 1);
    for (unsigned u = first; u < (unsigned)n_units; u += c.grid) {
        const float* slot_bias = nullptr;
        float acc[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[nt][e] = 0.f;
        for (int kc = 0; kc < p.n_kchunks; ++kc, ++consumed) {
            if (p.n_kchunks > 1) {
                consumer_sync();                       // everyone has finished with the chunk staged before
                stage_plain(c, op, p, kc * p.kchunk);
                consumer_sync();
            }
            const int slot = consumed % DP_SLOTS;
            if (!c.sh->abort_flag && !tbar_wait_or_abort(&c.sh->full[slot], (consumed / DP_SLOTS) & 1, &c.sh->abort_flag) &&
                lane == 0 && !c.sh->abort_flag)
                raise_abort(c);
            if (u == first && kc == 0) stamp(c, op_index, 2);
            const unsigned char* wt = c.ring + (size_t)slot * DP_SLOT_BYTES;
            if (kc == 0 && op.bias != nullptr && min(p.ncols, op.N - (int)u * p.ncols) % 4 == 0)
                slot_bias = reinterpret_cast<const float*>(wt + (size_t)p.ncols * p.w_stride);
            for (int piece = warp; piece < n_pieces; piece += DP_CONSUMER_WARPS) {
                const int kb = (piece * 32 + 8 * t) * 2;
                const uint4 a = *reinterpret_cast<const uint4*>(c.stage + (size_t)g * p.a_stride + kb);
                uint4 a8 = make_uint4(0u, 0u, 0u, 0u);
                if (high_rows) a8 = *reinterpret_cast<const uint4*>(c.stage + (size_t)(g + 8) * p.a_stride + kb);
                const uint4 b = *reinterpret_cast<const uint4*>(wt + (size_t)g * p.w_stride + kb);
                mma_16816(acc[0], a.x, a8.x, a.y, a8.y, b.x, b.y);
                mma_16816(acc[0], a.z, a8.z, a.w, a8.w, b.z, b.w);
                if (p.ncols == 16) {
                    const uint4 b2 = *reinterpret_cast<const uint4*>(wt + (size_t)(g + 8) * p.w_stride + kb);
                    mma_16816(acc[1], a.x, a8.x, a.y, a8.y, b2.x, b2.y);
                    mma_16816(acc[1], a.z, a8.z, a.w, a8.w, b2.z, b2.w);
                }
            }
            __syncwarp();
            if (lane == 0 && (kc > 0 || slot_bias == nullptr)) tbar_arrive(&c.sh->empty[slot]);
        }
        if (u == first) stamp(c, op_index, 3);
        const int bias_slot = (consumed - p.n_kchunks) % DP_SLOTS;     // the unit's first slot also holds its bias
        // the warps' partial tiles, added in the order of the warps
        float* mine = c.red + warp * 256;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            *reinterpret_cast<float2*>(mine + g * 16 + nt * 8 + 2 * t) = make_float2(acc[nt][0], acc[nt][1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * 16 + nt * 8 + 2 * t) = make_float2(acc[nt][2], acc[nt][3]);
        }
        consumer_sync();
        gemv_epilogue(c, op, p, u * p.ncols, slot_bias, u == first, residual_first);
        consumer_sync();
        if (slot_bias != nullptr && lane == 0) tbar_arrive(&c.sh->empty[bias_slot]);
    }
}

__device__ void run_embed(const Ctx& c, const DecodeOp& op, int op_index) {
    const unsigned rot = (unsigned)(op_index * 53) % c.grid;
    const int d = op.N;
    for (unsigned r = (blockIdx.x + c.grid - rot) % c.grid; r < (unsigned)c.n_rows; r += c.grid) {
        int tok = __ldcg(op.tokens + r), pos = c.sh->tok_pos[r];
        if (c.sh->tok_slot[r] < 0) { tok = 0; pos = 0; }
        if (tok < 0 || tok >= op.vocab) {
            if (threadIdx.x == 0) atomicOr(c.dev_err, VLRF_DEVERR_TOKEN_RANGE);
            tok = min(max(tok, 0), op.vocab - 1);
        }
        if (op.wpe != nullptr && (pos < 0 || pos >= op.n_pos)) {
            if (threadIdx.x == 0) atomicOr(c.dev_err, VLRF_DEVERR_POSITION_RANGE);
            pos = min(max(pos, 0), op.n_pos - 1);
        }
        const uint32_t* e = reinterpret_cast<const uint32_t*>(static_cast<const __nv_bfloat16*>(op.W) + (size_t)tok * d);
        const uint32_t* q = op.wpe == nullptr ? nullptr
            : reinterpret_cast<const uint32_t*>(static_cast<const __nv_bfloat16*>(op.wpe) + (size_t)pos * d);
        float* x = static_cast<float*>(op.out) + (size_t)r * op.ld_out;
        for (int i = threadIdx.x; i < d / 2; i += DP_CONSUMERS) {
            const uint32_t a = __ldg(e + i);
            float lo = bf_lo(a), hi = bf_hi(a);
            if (q != nullptr) {
                const uint32_t b = __ldg(q + i);
                lo += bf_lo(b);
                hi += bf_hi(b);
            }
            *reinterpret_cast<float2*>(x + 2 * i) = make_float2(lo, hi);
        }
    }
}

// ---- attention of one query per (row, head) over the paged cache ----
__device__ void run_attention(const Ctx& c, const DecodeOp& op, int op_index) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = op.n_heads, S = op.n_split, dh = op.dh;
    const int tpk = dh / 8, kpi = 32 / tpk;             // threads a key; keys a warp reads at once
    const int sub = lane % tpk, group = lane / tpk;
    const int n_units = c.n_rows * H * S;
    const unsigned rot = (unsigned)(op_index * 53) % c.grid;
    const int bt = op.bt, n_hkv = op.hkv, table_ld = op.table_ld;
    const int* op_table = op.table;
    const bool use_table = c.sh->table_of == op.table;
    float* wpart = reinterpret_cast<float*>(c.stage);   // [warps][dh + 2]
    const __nv_bfloat16* Kc = static_cast<const __nv_bfloat16*>(op.kc);
    const __nv_bfloat16* Vc = static_cast<const __nv_bfloat16*>(op.vc);
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(op.out);
    for (unsigned u = (blockIdx.x + c.grid - rot) % c.grid; u < (unsigned)n_units; u += c.grid) {
        const int b = u / (H * S), h = (u / S) % H, s = u % S;
        const int slot = c.sh->tok_slot[b], pos = c.sh->tok_pos[b];
        if (slot < 0) {                                   // a padding row: zeros, so that nothing downstream sees old bits
            if (s == 0)
                for (int j = threadIdx.x; j < dh; j += DP_CONSUMERS) out[(size_t)b * op.ld_out + h * dh + j] = __float2bfloat16_rn(0.f);
            continue;
        }
        const int n_keys = pos + 1;
        const int first = (op.window > 0 && n_keys > op.window) ? n_keys - op.window : 0;
        const int part = (((n_keys - first + S - 1) / S) + 31) & ~31;
        const int k_begin = first + s * part;
        const int k_end = min(n_keys, k_begin + part);
        const int hkv = h / (H / op.hkv);
        float q[8];
        {
            const uint4 w = ldcg_u4(static_cast<const __nv_bfloat16*>(op.in) + (size_t)b * op.ld_in + op.q_off + h * dh + 8 * sub);
            const float f = op.scale * 1.4426950408889634f;     // scores in base 2
            q[0] = bf_lo(w.x) * f; q[1] = bf_hi(w.x) * f; q[2] = bf_lo(w.y) * f; q[3] = bf_hi(w.y) * f;
            q[4] = bf_lo(w.z) * f; q[5] = bf_hi(w.z) * f; q[6] = bf_lo(w.w) * f; q[7] = bf_hi(w.w) * f;
        }
        float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        const int KB = kpi * DP_ATT_UNROLL;
        stamp(c, op_index, 1);
        for (int k0 = k_begin + warp * KB; k0 < k_end; k0 += DP_CONSUMER_WARPS * KB) {
            // every load asked for before any is used: no load is predicated (a key beyond the end reads the last
            // key again, an unmapped block reads block 0), what must not count is masked afterwards
            uint4 kr[DP_ATT_UNROLL], vr[DP_ATT_UNROLL];
            bool ok[DP_ATT_UNROLL];
            size_t at[DP_ATT_UNROLL];
            bool unmapped = false;
#pragma unroll
            for (int j = 0; j < DP_ATT_UNROLL; ++j) {
                const int kp = k0 + j * kpi + group;
                ok[j] = kp < k_end;
                const int kq = min(kp, k_end - 1);
                const int blk = use_table ? c.table[b * table_ld + kq / bt] : __ldg(op_table + (size_t)slot * table_ld + kq / bt);
                if (blk < 0 && ok[j]) { unmapped = true; ok[j] = false; }
                at[j] = (((size_t)max(blk, 0) * n_hkv + hkv) * bt + kq % bt) * dh + 8 * sub;
            }
#pragma unroll
            for (int j = 0; j < DP_ATT_UNROLL; ++j) kr[j] = ldcg_u4(Kc + at[j]);
#pragma unroll
            for (int j = 0; j < DP_ATT_UNROLL; ++j) vr[j] = ldcg_u4(Vc + at[j]);
            if (unmapped) atomicOr(c.dev_err, VLRF_DEVERR_NO_BLOCK);
            float sc[DP_ATT_UNROLL], mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < DP_ATT_UNROLL; ++j) {
                float d = q[0] * bf_lo(kr[j].x) + q[1] * bf_hi(kr[j].x) + q[2] * bf_lo(kr[j].y) + q[3] * bf_hi(kr[j].y)
                        + q[4] * bf_lo(kr[j].z) + q[5] * bf_hi(kr[j].z) + q[6] * bf_lo(kr[j].w) + q[7] * bf_hi(kr[j].w);
                for (int o = tpk >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                sc[j] = ok[j] ? d : -INFINITY;
                mx = fmaxf(mx, sc[j]);
            }
            if (mx > -INFINITY) {
                const float m_new = fmaxf(m, mx);
                const float corr = exp2f(m - m_new);          // m = −inf the first time: 0
                l *= corr;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] *= corr;
#pragma unroll
                for (int j = 0; j < DP_ATT_UNROLL; ++j) {
                    const float pj = exp2f(sc[j] - m_new);    // −inf for keys that are not there: 0
                    l += pj;
                    acc[0] += pj * bf_lo(vr[j].x); acc[1] += pj * bf_hi(vr[j].x);
                    acc[2] += pj * bf_lo(vr[j].y); acc[3] += pj * bf_hi(vr[j].y);
                    acc[4] += pj * bf_lo(vr[j].z); acc[5] += pj * bf_hi(vr[j].z);
                    acc[6] += pj * bf_lo(vr[j].w); acc[7] += pj * bf_hi(vr[j].w);
                }
                m = m_new;
            }
            if (k0 == k_begin + warp * KB) stamp(c, op_index, 2);
        }
        stamp(c, op_index, 3);
        // the groups of a warp, then the warps, then (through global memory) the parts: each in a fixed order
        for (int o = tpk; o < 32; o <<= 1) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
            const float mn = fmaxf(m, m2);
            const float c1 = mn > -INFINITY ? exp2f(m - mn) : 0.f, c2 = mn > -INFINITY ? exp2f(m2 - mn) : 0.f;
            l = l * c1 + l2 * c2;
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[e] = acc[e] * c1 + __shfl_xor_sync(0xffffffffu, acc[e], o) * c2;
            m = mn;
        }
        float* wp = wpart + warp * (dh + 2);
        if (group == 0) {
#pragma unroll
            for (int e = 0; e < 8; ++e) wp[2 + 8 * sub + e] = acc[e];
            if (sub == 0) { wp[0] = m; wp[1] = l; }
        }
        consumer_sync();
        const int j = threadIdx.x;
        float M = -INFINITY, L = 0.f, A = 0.f;
        if (j < dh) {
            for (int w = 0; w < DP_CONSUMER_WARPS; ++w) M = fmaxf(M, wpart[w * (dh + 2)]);
            for (int w = 0; w < DP_CONSUMER_WARPS; ++w) {
                const float mw = wpart[w * (dh + 2)];
                const float f = mw > -INFINITY ? exp2f(mw - M) : 0.f;
                L += wpart[w * (dh + 2) + 1] * f;
                A += wpart[w * (dh + 2) + 2 + j] * f;
            }
        }
        if (S == 1) {
            if (j < dh) out[(size_t)b * op.ld_out + h * dh + j] = __float2bfloat16_rn(L > 0.f ? A / L : 0.f);
            consumer_sync();
            continue;
        }
        const size_t pbase = ((size_t)b * H + h) * S;
        float* mine = op.partials + (pbase + s) * (dh + 2);
        if (j < dh) {
            mine[2 + j] = A;
            if (j == 0) { mine[0] = M; mine[1] = L; }
        }
        __threadfence();
        consumer_sync();
        if (threadIdx.x == 0) {
            const int old = atomicAdd(op.counters + (size_t)b * H + h, 1);
            c.sh->last_flag = old == S - 1;
        }
        consumer_sync();
        if (c.sh->last_flag) {
            __threadfence();
            if (j < dh) {
                float MM = -INFINITY, LL = 0.f, AA = 0.f;
                for (int z = 0; z < S; ++z) MM = fmaxf(MM, __ldcg(op.partials + (pbase + z) * (dh + 2)));
                for (int z = 0; z < S; ++z) {
                    const float* pz = op.partials + (pbase + z) * (dh + 2);
                    const float mz = __ldcg(pz);
                    const float f = mz > -INFINITY ? exp2f(mz - MM) : 0.f;
                    LL += __ldcg(pz + 1) * f;
                    AA += __ldcg(pz + 2 + j) * f;
                }
                out[(size_t)b * op.ld_out + h * dh + j] = __float2bfloat16_rn(LL > 0.f ? AA / LL : 0.f);
            }
            if (threadIdx.x == 0) op.counters[(size_t)b * H + h] = 0;
        }
        consumer_sync();
    }
}

__global__ void __launch_bounds__(DP_THREADS, 1)
decode_program_kernel(const DecodeOp* __restrict__ ops, int n_ops, int n_rows, const int* __restrict__ tok_slot,
                      const int* __restrict__ tok_pos, unsigned* __restrict__ sync_words, int* __restrict__ dev_err,
                      long long* __restrict__ trace) {
    extern __shared__ __align__(128) unsigned char smem[];
    Ctx c;
    c.ring = smem;
    c.stage = smem + DP_SLOTS * DP_SLOT_BYTES;
    c.red = reinterpret_cast<float*>(c.stage + DP_STAGE_BYTES);
    c.table = reinterpret_cast<int*>(c.red + DP_RED_FLOATS);
    c.sh = reinterpret_cast<Shared*>(c.table + DP_TABLE_INTS);
    c.sync_words = sync_words;
    c.dev_err = dev_err;
    c.trace = trace;
    c.trace_cta = trace != nullptr ? sync_words[3] % gridDim.x : 0u;
    c.n_rows = n_rows;
    c.grid = gridDim.x;
    const int tid = threadIdx.x;
    if (tid == 0) {
        for (int i = 0; i < DP_SLOTS; ++i) {
            tbar_init(&c.sh->full[i], 1);
            tbar_init(&c.sh->empty[i], DP_CONSUMER_WARPS);
        }
        c.sh->abort_flag = 0;
        c.sh->go_flag = 1;
        c.sh->last_flag = 0;
        c.sh->table_of = nullptr;
        c.sh->table_ld = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid >= 64 && tid < 64 + (int)(sizeof(DecodeOp) / 4))
        reinterpret_cast<uint32_t*>(&c.sh->op[0])[tid - 64] = reinterpret_cast<const uint32_t*>(ops)[tid - 64];
    if (tid < DP_MAX_ROWS) {
        c.sh->tok_slot[tid] = tid < n_rows ? tok_slot[tid] : -1;
        c.sh->tok_pos[tid] = tid < n_rows ? tok_pos[tid] : 0;
    }
    __syncthreads();
    // the block-table rows of this step's sequences, of the first operation that has a table
    for (int i = 0; i < n_ops; ++i) {
        if (ops[i].table == nullptr) continue;
        const int ld = ops[i].table_ld;
        if (n_rows * ld <= DP_TABLE_INTS) {
            for (int e = tid; e < n_rows * ld; e += DP_THREADS) {
                const int slot = c.sh->tok_slot[e / ld];
                c.table[e] = slot < 0 ? -1 : ops[i].table[(size_t)slot * ld + e % ld];
            }
            if (tid == 0) { c.sh->table_of = ops[i].table; c.sh->table_ld = ld; }
        }
        break;
    }
    __syncthreads();
    if (tid >= DP_CONSUMERS) {
        produce(c, ops, n_ops);
    } else {
        uint32_t consumed = 0;
        bool alive = true;
        for (int i = 0; i < n_ops && alive; ++i) {
            const DecodeOp& op = c.sh->op[i & 1];
            stamp(c, i, 0);
            if (op.kind == DP_EMBED) run_embed(c, op, i);
            else if (op.kind == DP_GEMV) run_gemv(c, op, i, consumed);
            else run_attention(c, op, i);
            if (i + 1 < n_ops) alive = grid_barrier(c, (unsigned)(i + 1) * c.grid, ops + i + 1, &c.sh->op[(i + 1) & 1]);
        }
        stamp(c, n_ops, 0);
    }
    __syncthreads();
    // the last CTA to leave puts the counters back for the next launch
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(sync_words + 1, 1u);
        if (old == gridDim.x - 1) {
            sync_words[0] = 0u;
            sync_words[2] = 0u;
            __threadfence();
            sync_words[1] = 0u;
        }
    }
}

constexpr size_t DP_SMEM_BYTES = (size_t)DP_SLOTS * DP_SLOT_BYTES + DP_STAGE_BYTES + DP_RED_FLOATS * 4 + DP_TABLE_INTS * 4 + sizeof(Shared);

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

extern "C" int vlrf_decode_program_op_bytes() { return (int)sizeof(DecodeOp); }
extern "C" int vlrf_decode_program_max_rows() { return DP_MAX_ROWS; }

extern "C" int vlrf_decode_program_gemv_takes(int n_rows, int N, int K, int in_f32, int norm) {
    GemvPlan p;
    if (n_rows < 1 || n_rows > DP_MAX_ROWS || N < 1 || !dp_plan_gemv(n_rows, K, &p)) return 0;
    if (p.n_kchunks > DP_SLOTS - 1) return 0;       // a unit's first slot is held (for its bias) until its last chunk is done
    if (norm != DP_NORM_NONE && (p.n_kchunks != 1 || K > DP_MAX_K_SINGLE || !in_f32)) return 0;
    return 1;
}

extern "C" int vlrf_decode_program_attention_takes(int head_dim, int block_tokens) {
    const bool dh_ok = head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
    return dh_ok && block_tokens > 0 && block_tokens % 32 == 0 ? 1 : 0;
}

extern "C" int vlrf_decode_op_embed(void* ops_host, int index, const void* wte, const void* wpe, const int* tokens, float* x,
                                    int d, int V, int P) {
    VLRF_REQUIRE(ops_host != nullptr && index >= 0 && wte != nullptr && tokens != nullptr && x != nullptr, "decode program: null argument");
    VLRF_REQUIRE(d > 0 && d % 2 == 0 && V > 0, "decode program: an embedding of width %d (even widths only)", d);
    DecodeOp op = {};
    op.kind = DP_EMBED;
    op.N = d; op.ld_out = d; op.vocab = V; op.n_pos = P;
    op.W = wte; op.wpe = wpe; op.tokens = tokens; op.out = x;
    static_cast<DecodeOp*>(ops_host)[index] = op;
    return VLRF_OK;
}

extern "C" int vlrf_decode_op_gemv(void* ops_host, int index, int n_rows, const void* in, int in_f32, int ld_in, int norm,
                                   const float* gamma, const float* beta, float eps, const void* W, const float* bias, int N,
                                   int K, int act, void* out, int out_f32, int ld_out, const float* residual, void* kc,
                                   void* vc, const int* block_table, int max_blocks, int k_off, int v_off, int Hkv, int dh,
                                   int BT) {
    VLRF_REQUIRE(ops_host != nullptr && index >= 0 && in != nullptr && W != nullptr && out != nullptr, "decode program: null argument");
    VLRF_REQUIRE(vlrf_decode_program_gemv_takes(n_rows, N, K, in_f32, norm),
                 "decode program: a product of %d rows, N=%d, K=%d (norm %d) is not taken: K a multiple of 32, at most %d rows, "
                 "a normed input float32 of at most %d columns", n_rows, N, K, norm, DP_MAX_ROWS, DP_MAX_K_SINGLE);
    VLRF_REQUIRE(aligned16(W) && aligned16(in) && aligned16(bias) && ld_in % 8 == 0 && ld_in >= K,
                 "decode program: operands must be 16-byte aligned");
    VLRF_REQUIRE(norm == DP_NORM_NONE || (gamma != nullptr && aligned16(gamma) && (beta == nullptr || aligned16(beta))),
                 "decode program: a norm needs its weight");
    VLRF_REQUIRE(ld_out >= N, "decode program: output rows are shorter than N");
    DecodeOp op = {};
    op.kind = DP_GEMV;
    op.N = N; op.K = K; op.in_f32 = in_f32; op.ld_in = ld_in; op.norm = norm; op.act = act; op.out_f32 = out_f32; op.ld_out = ld_out;
    op.eps = eps;
    op.in = in; op.gamma = gamma; op.beta = beta; op.W = W; op.bias = bias; op.out = out; op.residual = residual;
    if (kc != nullptr) {
        VLRF_REQUIRE(!out_f32 && vc != nullptr && block_table != nullptr && Hkv > 0 && dh > 0 && BT > 0 &&
                     k_off >= 0 && v_off >= 0 && k_off + Hkv * dh <= N && v_off + Hkv * dh <= N,
                     "decode program: the cache scatter does not match the projection");
        op.kc = kc; op.vc = vc; op.table = block_table; op.table_ld = max_blocks;
        op.k_off = k_off; op.v_off = v_off; op.hkv = Hkv; op.dh = dh; op.bt = BT;
    }
    static_cast<DecodeOp*>(ops_host)[index] = op;
    return VLRF_OK;
}

extern "C" int vlrf_decode_op_attention(void* ops_host, int index, const void* qkv, int ld_qkv, int q_off, const void* kc,
                                        const void* vc, const int* block_table, int max_blocks, void* out, int ld_out, int H,
                                        int Hkv, int dh, int BT, float scale, int window, int n_split, float* partials,
                                        int* counters) {
    VLRF_REQUIRE(ops_host != nullptr && index >= 0 && qkv != nullptr && kc != nullptr && vc != nullptr && block_table != nullptr &&
                 out != nullptr, "decode program: null argument");
    VLRF_REQUIRE(vlrf_decode_program_attention_takes(dh, BT), "decode program: attention with head size %d is not taken (16, 32, 64, 128, 256)", dh);
    VLRF_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0 && n_split >= 1, "decode program: heads do not match");
    VLRF_REQUIRE(n_split == 1 || (partials != nullptr && counters != nullptr), "decode program: parts need scratch");
    VLRF_REQUIRE(aligned16(qkv) && ld_qkv % 8 == 0 && q_off % 8 == 0 && aligned16(kc) && aligned16(vc),
                 "decode program: attention operands must be 16-byte aligned");
    DecodeOp op = {};
    op.kind = DP_ATTENTION;
    op.in = qkv; op.ld_in = ld_qkv; op.q_off = q_off; op.kc = const_cast<void*>(kc); op.vc = const_cast<void*>(vc);
    op.table = block_table; op.table_ld = max_blocks; op.out = out; op.ld_out = ld_out;
    op.n_heads = H; op.hkv = Hkv; op.dh = dh; op.bt = BT; op.scale = scale; op.window = window; op.n_split = n_split;
    op.partials = partials; op.counters = counters;
    static_cast<DecodeOp*>(ops_host)[index] = op;
    return VLRF_OK;
}

// Runs the operations (device array of vlrf_decode_program_op_bytes() each, filled on the host by the functions
// above and copied over) for n_rows rows whose slots and positions are tok_slot / tok_pos.  sync_words: 4 uint32
// on the device, zero before the first launch (the kernel leaves them zero).  One launch; launches that share
// sync_words, or scratch named in the operations, must not overlap.  trace: null, or int64 [n_ops + 1][8] on the
// device that receives times in nanoseconds of the CTA that sync_words[3] names: [op][0] the operation begins (and
// [n_ops][0]: the last has finished), [op][1…5] stages inside it.
extern "C" int vlrf_decode_program_run(const void* ops_dev, int n_ops, int n_rows, const int* tok_slot, const int* tok_pos,
                                       void* sync_words, int* dev_err, long long* trace, cudaStream_t stream) {
    VLRF_REQUIRE(ops_dev != nullptr && tok_slot != nullptr && tok_pos != nullptr && sync_words != nullptr && dev_err != nullptr,
                 "decode program: null argument");
    VLRF_REQUIRE(n_ops > 0 && n_rows >= 1 && n_rows <= DP_MAX_ROWS, "decode program: %d rows (at most %d)", n_rows, DP_MAX_ROWS);
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0, n = 0, coop = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess)
            return vlrf_fail(VLRF_ERR_CUDA, "decode program: cannot query the device");
        if (!coop) return vlrf_fail(VLRF_ERR_UNSUPPORTED, "decode program: the device has no cooperative launch");
        if (cudaFuncSetAttribute(decode_program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)DP_SMEM_BYTES) != cudaSuccess)
            return vlrf_check_launch("decode program (shared memory)");
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_program_kernel, DP_THREADS, DP_SMEM_BYTES) != cudaSuccess || per_sm < 1)
            return vlrf_fail(VLRF_ERR_UNSUPPORTED, "decode program: a CTA does not fit an SM");
        sm_count = n;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)sm_count);
    cfg.blockDim = dim3(DP_THREADS);
    cfg.dynamicSmemBytes = DP_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, decode_program_kernel, static_cast<const DecodeOp*>(ops_dev), n_ops, n_rows, tok_slot,
                                       tok_pos, static_cast<unsigned*>(sync_words), dev_err, trace);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "decode program: %s", cudaGetErrorString(e));
    return VLRF_OK;
}
