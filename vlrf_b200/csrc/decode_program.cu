// A whole decode step as ONE persistent kernel that runs a list of operations.
//
// A decode step of a small batch is a chain of some sixty tiny dependent operations (norm + projection,
// attention, projection + residual, ...).  As sixty launches each pays its own start-up, and none streams
// long enough to come near the memory rate.  Here one CTA per SM stays resident for the whole step and all CTAs
// walk the same list of operations.  What the list holds is decided by the model's parts on the host: this file
// knows three kinds of operation and no architecture.
//
//   EMBED      x[r] = wte[token[r]] + wpe[position[r]]                           float32 rows
//   GEMV       out[r] = act(norm(in[r]) · Wᵀ + bias) (+ residual[r])             few rows, W [N][K] bfloat16
//              norm: none, LayerNorm (two passes, float32) or RMS norm, applied while the rows are staged;
//              optionally the K and V columns of the result are also written into a paged cache
//   ATTENTION  one query per (row, head) over the keys 0…position of its slot in a paged cache,
//              float32 online softmax, the context cut into parts that the last CTA to finish merges in order
//
// There is no barrier between operations.  What one operation hands to the next (the residual rows, q/k/v, the
// merged heads, the inner rows of the feed-forward) lies in buffers whose every 8 bytes hold data AND a flag: one
// float32 and a 32-bit flag, or three bfloat16 and a 16-bit flag; the flag is the number of the (launch, operation)
// that wrote them.  A 64-bit store is single-copy atomic in the PTX memory model, so data and flag land together,
// and a reader that polls a group until its flag is the expected one has the data without any fence, counter or
// second round trip: an operation starts the moment the groups it reads have landed, about one trip to L2 after
// they were stored.  (A grid barrier costs a drain of the stores, an atomic and a poll:
// some 2 µs of round trips per operation, measured, against 3–5 MB of weights per operation that stream in 1 µs.)
// A buffer is rewritten only by an operation that cannot begin before every reader of the old contents has finished:
// between two writes of the same buffer lies an operation that every reader feeds and the writer waits for.
//
// Weights never depend on an earlier operation, so one warp of each CTA (the producer) streams this CTA's share
// of every operation's weights (and norm weights and biases) through a ring of shared-memory slots with bulk copies,
// as far ahead as the ring allows, across operation boundaries; HBM stays busy while the other eight warps wait for
// their inputs.  The products run on `mma.sync` (bfloat16 in, float32 accumulate) with the rows as the 16-row
// operand; a 16-byte shared-memory read feeds two MMAs through a permutation of k that both operands share.  A unit
// of work of a GEMV is 8, 16 or 24 output columns; the eight warps split k and add their partial tiles through
// shared memory in a fixed order, so results do not depend on timing.
//
// All CTAs must be resident at once (they wait for one another's data): the kernel is launched cooperatively with
// one CTA per SM.  Every wait is bounded; a wait that runs out sets VLRF_DEVERR_WAIT_TIMEOUT and a flag that makes
// every CTA run through the rest of the list without waiting.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int DP_CONSUMER_WARPS = 8;
constexpr int DP_CONSUMERS = 32 * DP_CONSUMER_WARPS;
constexpr int DP_THREADS = DP_CONSUMERS + 32;
constexpr int DP_MAX_ROWS = 16;
constexpr int DP_SLOT_BYTES = 40 * 1024;
constexpr int DP_SLOTS = 4;
constexpr int DP_STAGE_BYTES = 52224;               // 16 rows of 1,600 bfloat16 with their padding
constexpr int DP_RED_FLOATS = DP_CONSUMER_WARPS * 16 * 24;
constexpr int DP_TABLE_INTS = 512;
constexpr int DP_MAX_K_F32 = 1984;                  // float32 rows are staged whole, a row in the registers of a warp
constexpr uint32_t DP_POLL_LIMIT = 1u << 21;        // rounds of polling before a wait gives up
constexpr int DP_ATT_UNROLL = 8;
constexpr int DP_BIAS_BYTES = 96;                   // room behind a slot's weight rows for the bias of its columns
constexpr int DP_MAX_DH = 256;

enum { DP_EMBED = 0, DP_GEMV = 1, DP_ATTENTION = 2 };
enum { DP_NORM_NONE = 0, DP_NORM_LAYER = 1, DP_NORM_RMS = 2 };
// plain rows, or rows of 8-byte groups of (1 float32, 32-bit flag | 3 bfloat16, 16-bit flag)
enum { FMT_F32 = 0, FMT_BF16 = 1, FMT_LL_F32 = 2, FMT_LL_BF16 = 3 };

// A buffer of rows.  Plain: `ld` elements a row.  Flagged: `ld` groups a row (even, rows begin on 16 bytes); the
// columns of a row are cut into segments of `seg` columns, each `gps` groups (even), so that a segment (say, a head)
// is written by one CTA; `dep`: the operation that writes it before this one reads it (its number gives the flag).
struct Buf { void* p; int32_t fmt, ld, seg, gps, dep, pad; };

struct alignas(16) DecodeOp {
    int32_t kind, N, K, norm, act, n_units, ncols, kchunk, n_kchunks, w_stride, a_cols, a_stride;
    float eps, scale;
    int32_t k_off, v_off, hkv, dh, bt, table_ld, n_heads, q_off, n_split, window, vocab, n_pos;
    int32_t log2_dh, log2_bt;
    Buf in, out, res;
    const float* gamma;
    const float* beta;
    const void* W;
    const float* bias;
    void* kc;
    void* vc;
    const int* table;
    float* partials;
    int* counters;
    const void* wpe;
    const int* tokens;
};

__host__ __device__ inline int dp_pad_stride(int bytes) {   // row stride ≡ 64 (mod 128): 16-byte reads of 8 rows hit 32 banks
    return bytes + ((64 - bytes % 128) + 128) % 128;
}
__host__ __device__ inline int dp_per(int fmt) { return fmt == FMT_LL_F32 ? 1 : 3; }
__host__ __device__ inline bool dp_is_ll(int fmt) { return fmt >= FMT_LL_F32; }

// How a GEMV is cut (decided on the host, carried in the operation): `ncols` output columns a unit (24 where the
// output is flagged bfloat16, so that units end on group boundaries; else as many of 24, 16, 8 as still leave about a
// unit per SM), weight chunks of `kchunk` columns of k (multiples of 32) that fit a ring slot, and `a_cols` columns of
// the input staged at once: all of K where the staging area holds them at this number of rows, else one weight chunk
// at a time.
inline bool dp_plan_gemv(int n_rows, int N, int K, int in_fmt, int out_fmt, DecodeOp* op) {
    if (K <= 0 || K % 32 != 0 || N <= 0 || n_rows < 1 || n_rows > DP_MAX_ROWS) return false;
    const int rows_pad = n_rows <= 8 ? 8 : 16;
    const bool in_f32 = in_fmt == FMT_F32 || in_fmt == FMT_LL_F32;
    int ncols = 24;
    if (out_fmt != FMT_LL_BF16) {
        if (N / 24 < 90) ncols = 16;
        if (N / 16 < 90) ncols = 8;
    }
    int limit = ((DP_SLOT_BYTES - DP_BIAS_BYTES) / ncols - 128) / 2;
    limit -= limit % 32;
    int n = (K + limit - 1) / limit;
    while (K % (n * 32) != 0) ++n;
    if (rows_pad * dp_pad_stride(K * 2) <= DP_STAGE_BYTES) {
        op->a_cols = K;
    } else {
        // one weight chunk of the rows at a time: smaller chunks, until a chunk of the rows fits the staging area
        while (rows_pad * dp_pad_stride(K / n * 2) > DP_STAGE_BYTES && n < K / 32) {
            ++n;
            while (K % (n * 32) != 0) ++n;
        }
        op->a_cols = K / n;
    }
    op->ncols = ncols;
    op->n_kchunks = n;
    op->kchunk = K / n;
    op->w_stride = dp_pad_stride(op->kchunk * 2);
    op->n_units = (N + ncols - 1) / ncols;
    op->a_stride = dp_pad_stride(op->a_cols * 2);
    if (in_f32 && (op->a_cols != K || K > DP_MAX_K_F32)) return false;   // float32 rows are staged whole
    return true;
}

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(DP_CONSUMERS) : "memory"); }
__device__ __forceinline__ int ld_volatile_i32(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// One group (8 bytes) and two neighbouring groups (16 bytes, as a vector of two 64-bit elements: each element is
// read whole, whatever the hardware does with the vector).  A group's low word is data; its high word is the flag
// (float32 rows) or the third bfloat16 below a 16-bit flag.
__device__ __forceinline__ uint2 ld_ll(const void* p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return make_uint2((uint32_t)v, (uint32_t)(v >> 32));
}
__device__ __forceinline__ uint4 ld_ll2(const void* p) {
    unsigned long long a, b;
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4((uint32_t)a, (uint32_t)(a >> 32), (uint32_t)b, (uint32_t)(b >> 32));
}
__device__ __forceinline__ void st_ll(void* p, uint32_t lo, uint32_t hi) {
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"((unsigned long long)lo | ((unsigned long long)hi << 32)) : "memory");
}
__device__ __forceinline__ uint4 ldcg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(tsm(dst)), "l"(src), "r"(bytes), "r"(tsm(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_16(void* dst_shared, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(tsm(dst_shared)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float bf_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// The CTA's state, in shared memory: the functions below take it by reference and keep nothing of it in registers
// across calls (the kernel runs nine warps, which leaves 168 registers a thread; kept in one inlined body, the
// operations' state spilled to local memory, and with all of an SM's memory given to the ring local memory is L2).
struct Shared {
    uint64_t full[DP_SLOTS];
    uint64_t empty[DP_SLOTS];
    int abort_flag;      // a wait ran out somewhere: every later wait is skipped
    int last_flag;
    int table_ld;
    int n_rows;
    const int* table_of;
    unsigned char* ring;
    unsigned char* stage;
    float* red;
    int* table;
    unsigned* sync_words;    // [0] launches so far, [1] exit counter, [2] abort flag
    int* dev_err;
    long long* trace;
    int n_ops;
    uint32_t epoch_base;     // flags of this launch: epoch_base + operation number + 1
    unsigned grid;
    uint32_t consumed;       // ring slots the consumers have used so far
    int tok_slot[DP_MAX_ROWS];
    int tok_pos[DP_MAX_ROWS];
    DecodeOp op[2];      // the operation being run and the next one
};
typedef Shared Ctx;

// trace[cta][op][k], k = 0: the CTA begins the operation; 1: its rows are staged (attention: query staged); 2: its first
// weights have landed (attention: first keys used); 3: products done (attention: all keys used); 4: results stored.
constexpr int DP_TRACE_STAMPS = 8;
__device__ __forceinline__ void stamp(Ctx& c, int op_index, int k) {
    if (c.trace != nullptr && threadIdx.x == 0) c.trace[((size_t)blockIdx.x * (c.n_ops + 1) + op_index) * DP_TRACE_STAMPS + k] = global_ns();
}

__device__ __forceinline__ void raise_abort(Ctx& c) {
    c.abort_flag = 1;
    atomicOr(c.dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
    atomicExch(reinterpret_cast<int*>(c.sync_words + 2), 1);
}
// after a round of polling that did not find everything: whether to give up (another CTA did, or the limit is reached)
__device__ __forceinline__ bool poll_gives_up(Ctx& c, uint32_t& rounds) {
    ++rounds;
    if (c.abort_flag) return true;
    if ((rounds & 63u) == 0 && ld_volatile_i32(reinterpret_cast<const int*>(c.sync_words + 2))) {
        c.abort_flag = 1;
        return true;
    }
    if (rounds > DP_POLL_LIMIT) {
        raise_abort(c);
        return true;
    }
    return false;
}
__device__ __forceinline__ uint32_t epoch_of(Ctx& c, int op_number) { return c.epoch_base + (uint32_t)op_number + 1u; }
// the group that holds column `col` of a row of a flagged buffer
__device__ __forceinline__ int group_of(const Buf& b, int col) {
    const int per = dp_per(b.fmt);
    if (col < b.seg) return col / per;
    return (col / b.seg) * b.gps + (col % b.seg) / per;
}
// whether a group carries the expected flag (32 bits beside a float32, 16 bits beside three bfloat16)
__device__ __forceinline__ bool flag_ok_f32(uint32_t hi, uint32_t epoch) { return hi == epoch; }
__device__ __forceinline__ bool flag_ok_bf16(uint32_t hi, uint32_t epoch) { return (hi >> 16) == (epoch & 0xffffu); }
// one group, polled until its flag is the expected one
__device__ __forceinline__ uint2 wait_group(Ctx& c, const void* p, uint32_t epoch, bool f32) {
    uint2 v = ld_ll(p);
    uint32_t rounds = 0;
    while (!(f32 ? flag_ok_f32(v.y, epoch) : flag_ok_bf16(v.y, epoch)) && !poll_gives_up(c, rounds)) v = ld_ll(p);
    return v;
}

__device__ __forceinline__ int block_of(Ctx& c, const DecodeOp& op, int row, int slot, int block_index) {
    if (c.table_of == op.table) return c.table[row * c.table_ld + block_index];
    return __ldg(op.table + (size_t)slot * op.table_ld + block_index);
}

// ---- the producer warp: this CTA's weight tiles of every operation, in the order the consumers use them ----
__device__ __forceinline__ bool producer_slot(Ctx& c, uint32_t filled) {
    const uint32_t round = filled / DP_SLOTS;
    if (round > 0 && !tbar_wait_or_abort(&c.empty[filled % DP_SLOTS], (round - 1) & 1, &c.abort_flag)) {
        if ((threadIdx.x & 31) == 0 && !c.abort_flag) raise_abort(c);
        return false;
    }
    return true;
}
__device__ __noinline__ void produce(Ctx& c, const DecodeOp* __restrict__ ops, int n_ops) {
    const int lane = threadIdx.x & 31;
    uint32_t filled = 0;
    for (int i = 0; i < n_ops; ++i) {
        const DecodeOp& op = ops[i];
        if (op.kind != DP_GEMV) continue;
        const unsigned rot = (unsigned)(i * 53) % c.grid;
        const unsigned first = (blockIdx.x + c.grid - rot) % c.grid;
        if (first >= (unsigned)op.n_units) continue;
        const unsigned char* W = static_cast<const unsigned char*>(op.W);
        const int ncols = op.ncols, kchunk = op.kchunk, w_stride = op.w_stride, K = op.K;
        if (op.norm != DP_NORM_NONE) {
            // the norm's weight and bias, a slot of their own: [gamma K floats][beta K floats]
            if (!producer_slot(c, filled)) return;
            const int slot = filled % DP_SLOTS;
            unsigned char* dst = c.ring + (size_t)slot * DP_SLOT_BYTES;
            if (lane == 0) {
                tbar_expect_tx(&c.full[slot], (uint32_t)K * 4 * (op.beta != nullptr ? 2 : 1));
                bulk_g2s(dst, op.gamma, (uint32_t)K * 4, &c.full[slot]);
                if (op.beta != nullptr) bulk_g2s(dst + (size_t)K * 4, op.beta, (uint32_t)K * 4, &c.full[slot]);
            }
            __syncwarp();
            ++filled;
        }
        for (unsigned u = first; u < (unsigned)op.n_units; u += c.grid) {
            const int n0 = u * ncols;
            const int rows = min(ncols, op.N - n0);
            const bool with_bias = op.bias != nullptr && rows % 4 == 0;
            for (int kc = 0; kc < op.n_kchunks; ++kc, ++filled) {
                if (!producer_slot(c, filled)) return;
                const int slot = filled % DP_SLOTS;
                unsigned char* dst = c.ring + (size_t)slot * DP_SLOT_BYTES;
                const bool bias_here = with_bias && kc == 0;
                if (lane == 0) tbar_expect_tx(&c.full[slot], (uint32_t)rows * kchunk * 2 + (bias_here ? rows * 4 : 0));
                __syncwarp();
                if (lane < rows)
                    bulk_g2s(dst + (size_t)lane * w_stride, W + ((size_t)(n0 + lane) * K + (size_t)kc * kchunk) * 2,
                             (uint32_t)kchunk * 2, &c.full[slot]);
                if (lane == 31 && bias_here)
                    bulk_g2s(dst + (size_t)ncols * w_stride, op.bias + n0, (uint32_t)rows * 4, &c.full[slot]);
            }
        }
    }
}

// ---- staging the rows of a GEMV: norm in float32, result bfloat16 [rows][a_stride bytes] ----
// A warp takes a row (and the row eight further on) and keeps it in registers: NF float32 a lane.  Every load of a
// batch is asked for before the first is used (a loop of their own, addresses clamped instead of loads predicated):
// written the obvious way, each load was followed by its use and the round trips to L2 ran one after another.
// (`params`: the norm's weight, then its bias, in shared memory.)  Column of element e of lane's vector j:
// plain rows, 4 float32 a vector: 4 (lane + 32 j) + e; flagged rows, 2 groups a vector: 2 (lane + 32 j) + e.
template <int NJ, bool LL>
__device__ __noinline__ void stage_f32_t(Ctx& c, const DecodeOp& op, const float* params) {
    constexpr int EPV = LL ? 2 : 4;
    constexpr int BATCH = NJ <= 12 ? NJ : (NJ <= 16 ? 8 : (NJ <= 25 ? 9 : 8));   // vectors in flight at once (4 registers each)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int K = op.K, norm = op.norm;
    const int nv = K / EPV;
    const float eps = op.eps;
    const bool with_beta = op.beta != nullptr;
    const uint32_t epoch = LL ? epoch_of(c, op.in.dep) : 0u;
    const size_t row_bytes = LL ? (size_t)op.in.ld * 8 : (size_t)op.in.ld * 4;
    const int a_stride = op.a_stride;
    for (int r = warp; r < c.n_rows; r += DP_CONSUMER_WARPS) {
        const unsigned char* xr = static_cast<const unsigned char*>(op.in.p) + (size_t)r * row_bytes;
        float f[NJ][EPV];
#pragma unroll
        for (int j0 = 0; j0 < NJ; j0 += BATCH) {
            uint4 v[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j)
                if (j0 + j < NJ) v[j] = LL ? ld_ll2(xr + 16 * min(lane + 32 * (j0 + j), nv - 1)) : ldcg_u4(xr + 16 * min(lane + 32 * (j0 + j), nv - 1));
            if (LL) {
                uint32_t rounds = 0;
                for (;;) {
                    bool ok = true;
#pragma unroll
                    for (int j = 0; j < BATCH; ++j)
                        if (j0 + j < NJ) ok = ok && v[j].y == epoch && v[j].w == epoch;
                    if (__all_sync(0xffffffffu, ok) || poll_gives_up(c, rounds)) break;
#pragma unroll
                    for (int j = 0; j < BATCH; ++j)
                        if (j0 + j < NJ && (v[j].y != epoch || v[j].w != epoch)) v[j] = ld_ll2(xr + 16 * min(lane + 32 * (j0 + j), nv - 1));
                }
            }
#pragma unroll
            for (int j = 0; j < BATCH; ++j) {
                if (j0 + j < NJ) {
                    const bool in_row = lane + 32 * (j0 + j) < nv;
                    if (LL) {
                        f[j0 + j][0] = in_row ? __uint_as_float(v[j].x) : 0.f;
                        f[j0 + j][1] = in_row ? __uint_as_float(v[j].z) : 0.f;
                    } else {
                        f[j0 + j][0] = in_row ? __uint_as_float(v[j].x) : 0.f;
                        f[j0 + j][1] = in_row ? __uint_as_float(v[j].y) : 0.f;
                        f[j0 + j][EPV - 2] = in_row ? __uint_as_float(v[j].z) : 0.f;
                        f[j0 + j][EPV - 1] = in_row ? __uint_as_float(v[j].w) : 0.f;
                    }
                }
            }
        }
        float mean = 0.f, rstd = 1.f;
        if (norm == DP_NORM_LAYER) {
            float sum = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j)
#pragma unroll
                for (int e = 0; e < EPV; ++e) sum += f[j][e];
            mean = warp_sum(sum) / (float)K;
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                if (lane + 32 * j < nv) {
#pragma unroll
                    for (int e = 0; e < EPV; ++e) sq += (f[j][e] - mean) * (f[j][e] - mean);
                }
            }
            rstd = rsqrtf(warp_sum(sq) / (float)K + eps);
        } else if (norm == DP_NORM_RMS) {
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < NJ; ++j)
#pragma unroll
                for (int e = 0; e < EPV; ++e) sq += f[j][e] * f[j][e];
            rstd = rsqrtf(warp_sum(sq) / (float)K + eps);
        }
        unsigned char* row = c.stage + (size_t)r * a_stride;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const int col0 = (lane + 32 * j) * EPV;
            if (col0 < K) {
                float y[EPV];
#pragma unroll
                for (int e = 0; e < EPV; ++e) {
                    y[e] = (f[j][e] - mean) * rstd;
                    if (norm != DP_NORM_NONE) {
                        y[e] *= params[col0 + e];
                        if (with_beta) y[e] += params[K + col0 + e];
                    }
                }
                if (LL) {
                    *reinterpret_cast<uint32_t*>(row + 2 * col0) = pack2(y[0], y[1]);
                } else {
                    uint2 o;
                    o.x = pack2(y[0], y[1]);
                    o.y = pack2(y[EPV - 2], y[EPV - 1]);
                    *reinterpret_cast<uint2*>(row + 2 * col0) = o;
                }
            }
        }
    }
}
template <bool LL>
__device__ __forceinline__ void stage_f32(Ctx& c, const DecodeOp& op, const float* params) {
    const int nj = (op.K / (LL ? 2 : 4) + 31) / 32;
    if (nj <= 4) stage_f32_t<4, LL>(c, op, params);
    else if (nj <= 8) stage_f32_t<8, LL>(c, op, params);
    else if (nj <= 12) stage_f32_t<12, LL>(c, op, params);
    else if (nj <= 16) stage_f32_t<16, LL>(c, op, params);
    else if (nj <= 25) stage_f32_t<25, LL>(c, op, params);
    else stage_f32_t<31, LL>(c, op, params);
}

// bfloat16 rows, columns [k0, k0 + a_cols): plain rows are copied asynchronously, all pieces in flight at once;
// of flagged rows a warp takes a row (and the row eight further on), eight vectors of two groups a lane in flight.
__device__ __noinline__ void stage_bf16(Ctx& c, const DecodeOp& op, int k0) {
    const int tid = threadIdx.x;
    const int a_stride = op.a_stride, a_cols = op.a_cols;
    if (op.in.fmt == FMT_BF16) {
        const int pieces = a_cols / 8;                    // 16-byte pieces a row
        const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(op.in.p) + k0;
        for (int i = tid; i < c.n_rows * pieces; i += DP_CONSUMERS) {
            const int r = i / pieces, q = i % pieces;
            cp_async_16(c.stage + (size_t)r * a_stride + 16 * q, src + (size_t)r * op.in.ld + 8 * q);
        }
        cp_async_wait_all();
        return;
    }
    // the vectors (pairs of groups) that hold columns k0 … k0 + a_cols − 1; a vector at the edge of the chunk is
    // read by both chunks and each keeps its own columns; a segment's last vector may hold one group only
    const int warp = tid >> 5, lane = tid & 31;
    const uint32_t epoch = epoch_of(c, op.in.dep);
    const int seg = op.in.seg, gps = op.in.gps, K = op.K;
    const int v_first = group_of(op.in, k0) >> 1, v_last = group_of(op.in, k0 + a_cols - 1) >> 1;
    const int vps = gps >> 1;                             // vectors a segment
    constexpr int INFLIGHT = 8;
    for (int r = warp; r < c.n_rows; r += DP_CONSUMER_WARPS) {
        const unsigned char* xr = static_cast<const unsigned char*>(op.in.p) + (size_t)r * op.in.ld * 8;
        uint16_t* row = reinterpret_cast<uint16_t*>(c.stage + (size_t)r * a_stride);
        for (int base = v_first; base <= v_last; base += 32 * INFLIGHT) {
            uint4 v[INFLIGHT];
#pragma unroll
            for (int j = 0; j < INFLIGHT; ++j) v[j] = ld_ll2(xr + 16 * min(base + lane + 32 * j, v_last));
            // which of a vector's two groups hold columns of the row: the second may lie beyond its segment's end
            bool second[INFLIGHT];
            int col0[INFLIGHT];
#pragma unroll
            for (int j = 0; j < INFLIGHT; ++j) {
                const int vi = min(base + lane + 32 * j, v_last);
                const int sg = vi < vps ? 0 : vi / vps;
                col0[j] = sg * seg + (vi - sg * vps) * 6;
                second[j] = col0[j] + 3 < min(K, (sg + 1) * seg);
            }
            uint32_t rounds = 0;
            for (;;) {
                bool ok = true;
#pragma unroll
                for (int j = 0; j < INFLIGHT; ++j) ok = ok && flag_ok_bf16(v[j].y, epoch) && (!second[j] || flag_ok_bf16(v[j].w, epoch));
                if (__all_sync(0xffffffffu, ok) || poll_gives_up(c, rounds)) break;
#pragma unroll
                for (int j = 0; j < INFLIGHT; ++j)
                    if (!flag_ok_bf16(v[j].y, epoch) || (second[j] && !flag_ok_bf16(v[j].w, epoch)))
                        v[j] = ld_ll2(xr + 16 * min(base + lane + 32 * j, v_last));
            }
#pragma unroll
            for (int j = 0; j < INFLIGHT; ++j) {
                if (base + lane + 32 * j > v_last) continue;
                const int seg_end = min(K, (col0[j] / seg + 1) * seg);
                const uint16_t e[6] = {(uint16_t)v[j].x, (uint16_t)(v[j].x >> 16), (uint16_t)v[j].y,
                                       (uint16_t)v[j].z, (uint16_t)(v[j].z >> 16), (uint16_t)v[j].w};
                if (col0[j] >= k0 && col0[j] + 6 <= k0 + a_cols && col0[j] + 6 <= seg_end) {
                    uint32_t* dst = reinterpret_cast<uint32_t*>(row + (col0[j] - k0));
                    dst[0] = v[j].x;
                    dst[1] = (uint32_t)e[2] | ((uint32_t)e[3] << 16);
                    dst[2] = (uint32_t)e[4] | ((uint32_t)e[5] << 16);
                } else {
#pragma unroll
                    for (int k = 0; k < 6; ++k) {
                        const int col = col0[j] + k;
                        if (col >= k0 && col < k0 + a_cols && col < seg_end) row[col - k0] = e[k];
                    }
                }
            }
        }
    }
}

__device__ __forceinline__ float finish_value(const DecodeOp& op, float v) {
    if (op.act == VLRF_ACT_GELU_TANH) return (op.out.fmt == FMT_F32 || op.out.fmt == FMT_LL_F32) ? gelu_tanh_f(v) : gelu_tanh_fast(v);
    if (op.act == VLRF_ACT_GELU_ERF) return gelu_erf_f(v);
    return v;
}
__device__ __forceinline__ void scatter_kv(Ctx& c, const DecodeOp& op, int r, int n, __nv_bfloat16 o) {
    const int width = op.hkv << op.log2_dh;
    __nv_bfloat16* cache;
    int col;
    if (n >= op.k_off && n < op.k_off + width) { cache = static_cast<__nv_bfloat16*>(op.kc); col = n - op.k_off; }
    else if (n >= op.v_off && n < op.v_off + width) { cache = static_cast<__nv_bfloat16*>(op.vc); col = n - op.v_off; }
    else return;
    const int slot = c.tok_slot[r], pos = c.tok_pos[r];
    if (slot < 0) return;
    const int blk = block_of(c, op, r, slot, pos >> op.log2_bt);
    if (blk < 0) { atomicOr(c.dev_err, VLRF_DEVERR_NO_BLOCK); return; }
    const size_t token = (((size_t)blk * op.hkv + (col >> op.log2_dh)) << op.log2_bt) + (pos & (op.bt - 1));
    cache[(token << op.log2_dh) + (col & (op.dh - 1))] = o;
}

// The results of a unit: a warp takes a row (and the row eight further on), a lane a column: the warps' partial
// tiles added in the order of the warps, bias, activation, residual, and the store (plain elements, or groups with
// their flag: a float32 each, or three bfloat16 gathered from three lanes).  `bias_l`: the bias of this lane's column.
__device__ __forceinline__ void gemv_epilogue(Ctx& c, const DecodeOp& op, int op_index, int n0, float bias_l, bool have_res,
                                              const uint2& res_first) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ncols = op.ncols, fmt = op.out.fmt, N = op.N;
    const int n = n0 + lane;
    const bool mine = lane < ncols && n < N;
    const uint32_t epoch = epoch_of(c, op_index);
    for (int r = warp; r < c.n_rows; r += DP_CONSUMER_WARPS) {
        float v = 0.f;
        if (mine) {
#pragma unroll
            for (int w = 0; w < DP_CONSUMER_WARPS; ++w) v += c.red[(w * 16 + r) * 24 + lane];
            v = finish_value(op, v + bias_l);
            if (op.res.p != nullptr) {
                if (fmt == FMT_LL_F32) {
                    const uint32_t want = epoch_of(c, op.res.dep);
                    uint2 old = res_first;
                    if (!(have_res && r == warp && old.y == want))
                        old = wait_group(c, static_cast<const unsigned char*>(op.res.p) + ((size_t)r * op.res.ld + n) * 8, want, true);
                    v += __uint_as_float(old.x);
                } else {
                    v += __ldcg(static_cast<const float*>(op.res.p) + (size_t)r * op.res.ld + n);
                }
            }
        }
        if (fmt == FMT_LL_BF16) {
            // three neighbouring lanes hold a group (units begin on group boundaries)
            const float v1 = __shfl_down_sync(0xffffffffu, v, 1), v2 = __shfl_down_sync(0xffffffffu, v, 2);
            if (mine && lane % 3 == 0) {
                const uint32_t lo = pack2(v, n + 1 < N ? v1 : 0.f);
                const uint32_t hi = (pack2(n + 2 < N ? v2 : 0.f, 0.f) & 0xffffu) | (epoch << 16);
                st_ll(static_cast<unsigned char*>(op.out.p) + ((size_t)r * op.out.ld + n / 3) * 8, lo, hi);
            }
            if (mine && op.kc != nullptr) scatter_kv(c, op, r, n, __float2bfloat16_rn(v));
        } else if (mine) {
            if (fmt == FMT_LL_F32) {
                st_ll(static_cast<unsigned char*>(op.out.p) + ((size_t)r * op.out.ld + n) * 8, __float_as_uint(v), epoch);
            } else if (fmt == FMT_F32) {
                static_cast<float*>(op.out.p)[(size_t)r * op.out.ld + n] = v;
            } else {
                const __nv_bfloat16 o = __float2bfloat16_rn(v);
                static_cast<__nv_bfloat16*>(op.out.p)[(size_t)r * op.out.ld + n] = o;
                if (op.kc != nullptr) scatter_kv(c, op, r, n, o);
            }
        }
    }
}

// No thread leaves an operation early: a wait that runs out raises the abort flag and the thread goes on (with
// meaningless numbers), so that the CTA's barriers always see all their threads.
__device__ __noinline__ void run_gemv(Ctx& c, const DecodeOp& op, int op_index) {
    uint32_t consumed = c.consumed;        // (every consumer thread computes the same count; one writes it back)
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const unsigned rot = (unsigned)(op_index * 53) % c.grid;
    const unsigned first = (blockIdx.x + c.grid - rot) % c.grid;
    if (first >= (unsigned)op.n_units) return;
    const int ncols = op.ncols, n_nt = ncols >> 3, N = op.N;
    const bool high_rows = c.n_rows > 8;
    const int kchunk = op.kchunk, n_kchunks = op.n_kchunks, n_pieces = kchunk / 32;
    const int a_stride = op.a_stride, w_stride = op.w_stride;
    // the residual of this lane's result of the first unit (row = warp): asked for now, used in the epilogue
    uint2 res_first = make_uint2(0u, 0u);
    const bool res_early = op.res.p != nullptr && op.out.fmt == FMT_LL_F32 && warp < c.n_rows && lane < ncols &&
                           (int)first * ncols + lane < N;
    if (res_early)
        res_first = ld_ll(static_cast<const unsigned char*>(op.res.p) + ((size_t)warp * op.res.ld + first * ncols + lane) * 8);
    const float* params = nullptr;
    int param_slot = -1;
    if (op.norm != DP_NORM_NONE) {
        param_slot = consumed % DP_SLOTS;
        if (!c.abort_flag && !tbar_wait_or_abort(&c.full[param_slot], (consumed / DP_SLOTS) & 1, &c.abort_flag) &&
            lane == 0 && !c.abort_flag)
            raise_abort(c);
        params = reinterpret_cast<const float*>(c.ring + (size_t)param_slot * DP_SLOT_BYTES);
        ++consumed;
    }
    const bool whole = op.a_cols == op.K;
    if (whole) {
        if (op.in.fmt == FMT_LL_F32) stage_f32<true>(c, op, params);
        else if (op.in.fmt == FMT_F32) stage_f32<false>(c, op, params);
        else stage_bf16(c, op, 0);
        consumer_sync();
    }
    if (param_slot >= 0 && lane == 0) tbar_arrive(&c.empty[param_slot]);
    stamp(c, op_index, 1);
    for (unsigned u = first; u < (unsigned)op.n_units; u += c.grid) {
        const int n0 = u * ncols;
        const bool bias_in_slot = op.bias != nullptr && min(ncols, N - n0) % 4 == 0;
        float bias_l = 0.f;
        float acc[3][2][4];
#pragma unroll
        for (int nt = 0; nt < 3; ++nt)
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[nt][h][e] = 0.f;
        for (int kc = 0; kc < n_kchunks; ++kc, ++consumed) {
            if (!whole) {
                consumer_sync();                       // everyone has finished with the chunk staged before
                stage_bf16(c, op, kc * kchunk);
                consumer_sync();
            }
            const int slot = consumed % DP_SLOTS;
            if (!c.abort_flag && !tbar_wait_or_abort(&c.full[slot], (consumed / DP_SLOTS) & 1, &c.abort_flag) &&
                lane == 0 && !c.abort_flag)
                raise_abort(c);
            if (u == first && kc == 0) stamp(c, op_index, 2);
            const unsigned char* wt = c.ring + (size_t)slot * DP_SLOT_BYTES;
            if (kc == 0 && op.bias != nullptr && lane < ncols && n0 + lane < N)     // kept in a register: the slot is given back below
                bias_l = bias_in_slot ? reinterpret_cast<const float*>(wt + (size_t)ncols * w_stride)[lane] : __ldg(op.bias + n0 + lane);
            const unsigned char* a_base = c.stage + (whole ? (size_t)kc * kchunk * 2 : 0);
            for (int piece = warp; piece < n_pieces; piece += DP_CONSUMER_WARPS) {
                const int kb = (piece * 32 + 8 * t) * 2;
                const uint4 a = *reinterpret_cast<const uint4*>(a_base + (size_t)g * a_stride + kb);
                uint4 a8 = make_uint4(0u, 0u, 0u, 0u);
                if (high_rows) a8 = *reinterpret_cast<const uint4*>(a_base + (size_t)(g + 8) * a_stride + kb);
#pragma unroll
                for (int nt = 0; nt < 3; ++nt) {
                    if (nt < n_nt) {
                        const uint4 b = *reinterpret_cast<const uint4*>(wt + (size_t)(nt * 8 + g) * w_stride + kb);
                        mma_16816(acc[nt][0], a.x, a8.x, a.y, a8.y, b.x, b.y);
                        mma_16816(acc[nt][1], a.z, a8.z, a.w, a8.w, b.z, b.w);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) tbar_arrive(&c.empty[slot]);
        }
        if (u == first) stamp(c, op_index, 3);
        // the warps' partial tiles, added in the order of the warps
        float* mine = c.red + warp * (16 * 24);
#pragma unroll
        for (int nt = 0; nt < 3; ++nt) {
            if (nt < n_nt) {
                *reinterpret_cast<float2*>(mine + g * 24 + nt * 8 + 2 * t) =
                    make_float2(acc[nt][0][0] + acc[nt][1][0], acc[nt][0][1] + acc[nt][1][1]);
                *reinterpret_cast<float2*>(mine + (g + 8) * 24 + nt * 8 + 2 * t) =
                    make_float2(acc[nt][0][2] + acc[nt][1][2], acc[nt][0][3] + acc[nt][1][3]);
            }
        }
        consumer_sync();
        gemv_epilogue(c, op, op_index, n0, bias_l, res_early && u == first, res_first);
        consumer_sync();
    }
    if (threadIdx.x == 0) c.consumed = consumed;     // (read again after the CTA barrier that ends the operation)
    stamp(c, op_index, 4);
}

__device__ __noinline__ void run_embed(Ctx& c, const DecodeOp& op, int op_index) {
    const unsigned rot = (unsigned)(op_index * 53) % c.grid;
    const int d = op.N;
    const __nv_bfloat16* wte = static_cast<const __nv_bfloat16*>(op.W);
    const __nv_bfloat16* wpe = static_cast<const __nv_bfloat16*>(op.wpe);
    for (unsigned r = (blockIdx.x + c.grid - rot) % c.grid; r < (unsigned)c.n_rows; r += c.grid) {
        int tok = __ldcg(op.tokens + r), pos = c.tok_pos[r];
        if (c.tok_slot[r] < 0) { tok = 0; pos = 0; }
        if (tok < 0 || tok >= op.vocab) {
            if (threadIdx.x == 0) atomicOr(c.dev_err, VLRF_DEVERR_TOKEN_RANGE);
            tok = min(max(tok, 0), op.vocab - 1);
        }
        if (wpe != nullptr && (pos < 0 || pos >= op.n_pos)) {
            if (threadIdx.x == 0) atomicOr(c.dev_err, VLRF_DEVERR_POSITION_RANGE);
            pos = min(max(pos, 0), op.n_pos - 1);
        }
        const __nv_bfloat16* e = wte + (size_t)tok * d;
        const __nv_bfloat16* q = wpe == nullptr ? nullptr : wpe + (size_t)pos * d;
        if (op.out.fmt == FMT_LL_F32) {
            unsigned char* x = static_cast<unsigned char*>(op.out.p) + (size_t)r * op.out.ld * 8;
            const uint32_t epoch = epoch_of(c, op_index);
            for (int i = threadIdx.x; i < d; i += DP_CONSUMERS)
                st_ll(x + (size_t)i * 8, __float_as_uint(__bfloat162float(e[i]) + (q != nullptr ? __bfloat162float(q[i]) : 0.f)), epoch);
        } else {
            float* x = static_cast<float*>(op.out.p) + (size_t)r * op.out.ld;
            for (int i = threadIdx.x; i < d; i += DP_CONSUMERS)
                x[i] = __bfloat162float(e[i]) + (q != nullptr ? __bfloat162float(q[i]) : 0.f);
        }
    }
}

// ---- attention of one query per (row, head) over the paged cache ----
// With a flagged q/k/v input (inside a step) the newest key and value are taken from that buffer, where the
// projection has just put them, and the cache is read up to the position before; with a plain input the cache
// holds every key.
__device__ __noinline__ void run_attention(Ctx& c, const DecodeOp& op, int op_index) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = op.n_heads, S = op.n_split, dh = op.dh;
    const int tpk = dh / 8, kpi = 32 / tpk;             // threads a key; keys a warp reads at once
    const int sub = lane % tpk, group = lane / tpk;
    const int n_units = c.n_rows * H * S;
    const unsigned rot = (unsigned)(op_index * 53) % c.grid;
    const int bt = op.bt, log2_bt = op.log2_bt, n_hkv = op.hkv, table_ld = op.table_ld;
    const int* op_table = op.table;
    const bool use_table = c.table_of == op.table;
    const bool ll_in = op.in.fmt == FMT_LL_BF16;
    float* wpart = reinterpret_cast<float*>(c.stage);   // [warps][dh + 2], then the merged output [dh]
    float* outs = wpart + DP_CONSUMER_WARPS * (dh + 2);
    float* qs = outs + dh;                              // this unit's query, then its newest key and value, [3][dh]
    const __nv_bfloat16* Kc = static_cast<const __nv_bfloat16*>(op.kc);
    const __nv_bfloat16* Vc = static_cast<const __nv_bfloat16*>(op.vc);
    const float qf = op.scale * 1.4426950408889634f;    // scores in base 2
    for (unsigned u = (blockIdx.x + c.grid - rot) % c.grid; u < (unsigned)n_units; u += c.grid) {
        const int b = u / (H * S), h = (u / S) % H, s = u % S;
        const int slot = c.tok_slot[b], pos = c.tok_pos[b];
        const int hkv = h / (H / n_hkv);
        const bool padding = slot < 0;
        // the query (and with a flagged input the newest key and value) of this (row, head), in shared memory
        if (ll_in) {
            const uint32_t epoch = epoch_of(c, op.in.dep);
            const int gmax = dh / 3 + 2;                      // groups that can hold a head's columns
            for (int i = threadIdx.x; i < 3 * gmax; i += DP_CONSUMERS) {
                const int which = i / gmax;
                const int c0 = which == 0 ? op.q_off + h * dh : (which == 1 ? op.k_off + hkv * dh : op.v_off + hkv * dh);
                const int gi = group_of(op.in, c0) + i % gmax;
                if (gi <= group_of(op.in, c0 + dh - 1)) {
                    const uint2 v = wait_group(c, static_cast<const unsigned char*>(op.in.p) + ((size_t)b * op.in.ld + gi) * 8, epoch, false);
                    const float e[3] = {bf_lo(v.x), bf_hi(v.x), bf_lo(v.y)};
#pragma unroll
                    for (int k = 0; k < 3; ++k) {
                        const int col = gi * 3 + k - c0;
                        if (col >= 0 && col < dh) qs[which * dh + col] = e[k];
                    }
                }
            }
        } else if ((int)threadIdx.x < dh) {
            qs[threadIdx.x] = __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(op.in.p) + (size_t)b * op.in.ld + op.q_off + h * dh + threadIdx.x));
        }
        consumer_sync();
        stamp(c, op_index, 1);
        const int n_cached = padding ? 0 : (ll_in ? pos : pos + 1);     // keys to read from the cache
        const int n_keys = padding ? 0 : pos + 1;
        const int first = (op.window > 0 && n_keys > op.window) ? n_keys - op.window : 0;
        const int part = (((max(n_cached - first, 0) + S - 1) / S) + 31) & ~31;
        const int k_begin = first + s * part;
        const int k_end = min(n_cached, k_begin + part);
        float q[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) q[e] = qs[8 * sub + e] * qf;
        float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] = 0.f;
        const int KB = kpi * DP_ATT_UNROLL;
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
                const int blk = use_table ? c.table[b * table_ld + (kq >> log2_bt)] : __ldg(op_table + (size_t)slot * table_ld + (kq >> log2_bt));
                if (blk < 0 && ok[j]) { unmapped = true; ok[j] = false; }
                at[j] = ((((size_t)max(blk, 0) * n_hkv + hkv) << log2_bt) + (kq & (bt - 1))) * dh + 8 * sub;
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
        if (ll_in && !padding && s == S - 1 && warp == 0) {
            // the newest key, from the projection's output: counted once, by the first group of the first warp
            float d = 0.f;
#pragma unroll
            for (int e = 0; e < 8; ++e) d += q[e] * qs[dh + 8 * sub + e];
            for (int o = tpk >> 1; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            if (group == 0) {
                const float m_new = fmaxf(m, d);
                const float corr = exp2f(m - m_new), pj = exp2f(d - m_new);
                l = l * corr + pj;
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[e] = acc[e] * corr + pj * qs[2 * dh + 8 * sub + e];
                m = m_new;
            }
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
        bool write_out = true;           // whether this CTA holds the (row, head)'s final output (in `outs`)
        if (S == 1 || padding) {
            if (j < dh) outs[j] = L > 0.f ? A / L : 0.f;
            write_out = S == 1 || s == 0;
        } else {
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
                c.last_flag = old == S - 1;
            }
            consumer_sync();
            write_out = c.last_flag != 0;
            if (write_out) {
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
                    outs[j] = LL > 0.f ? AA / LL : 0.f;
                }
                if (threadIdx.x == 0) op.counters[(size_t)b * H + h] = 0;
            }
        }
        consumer_sync();
        if (write_out) {
            if (op.out.fmt == FMT_LL_BF16) {
                const int gps = op.out.gps;      // the head is a segment of the output row
                if (3 * j < dh) {
                    const float v0 = outs[3 * j], v1 = 3 * j + 1 < dh ? outs[3 * j + 1] : 0.f, v2 = 3 * j + 2 < dh ? outs[3 * j + 2] : 0.f;
                    st_ll(static_cast<unsigned char*>(op.out.p) + ((size_t)b * op.out.ld + (size_t)h * gps + j) * 8,
                          pack2(v0, v1), (pack2(v2, 0.f) & 0xffffu) | (epoch_of(c, op_index) << 16));
                }
            } else if (j < dh) {
                static_cast<__nv_bfloat16*>(op.out.p)[(size_t)b * op.out.ld + h * dh + j] = __float2bfloat16_rn(outs[j]);
            }
        }
        consumer_sync();
    }
    stamp(c, op_index, 4);
}

__global__ void __launch_bounds__(DP_THREADS, 1)
decode_program_kernel(const DecodeOp* __restrict__ ops, int n_ops, int n_rows, const int* __restrict__ tok_slot,
                      const int* __restrict__ tok_pos, unsigned* __restrict__ sync_words, int* __restrict__ dev_err,
                      long long* __restrict__ trace) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* stage_at = smem + DP_SLOTS * DP_SLOT_BYTES;
    float* red_at = reinterpret_cast<float*>(stage_at + DP_STAGE_BYTES);
    int* table_at = reinterpret_cast<int*>(red_at + DP_RED_FLOATS);
    Ctx& c = *reinterpret_cast<Shared*>(table_at + DP_TABLE_INTS);
    const int tid = threadIdx.x;
    if (tid == 0) {
        c.ring = smem;
        c.stage = stage_at;
        c.red = red_at;
        c.table = table_at;
        c.sync_words = sync_words;
        c.dev_err = dev_err;
        c.trace = trace;
        c.n_ops = n_ops;
        c.epoch_base = sync_words[0] * (uint32_t)n_ops;       // (changed only by the last CTA of a launch to leave)
        c.n_rows = n_rows;
        c.grid = gridDim.x;
        c.consumed = 0;
        for (int i = 0; i < DP_SLOTS; ++i) {
            tbar_init(&c.full[i], 1);
            tbar_init(&c.empty[i], DP_CONSUMER_WARPS);
        }
        c.abort_flag = 0;
        c.last_flag = 0;
        c.table_of = nullptr;
        c.table_ld = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (tid >= 64 && tid < 64 + (int)(sizeof(DecodeOp) / 4))
        reinterpret_cast<uint32_t*>(&c.op[0])[tid - 64] = reinterpret_cast<const uint32_t*>(ops)[tid - 64];
    if (tid < DP_MAX_ROWS) {
        c.tok_slot[tid] = tid < n_rows ? tok_slot[tid] : -1;
        c.tok_pos[tid] = tid < n_rows ? tok_pos[tid] : 0;
    }
    __syncthreads();
    // the block-table rows of this step's sequences, of the first operation that has a table
    for (int i = 0; i < n_ops; ++i) {
        if (ops[i].table == nullptr) continue;
        const int ld = ops[i].table_ld;
        if (n_rows * ld <= DP_TABLE_INTS) {
            for (int e = tid; e < n_rows * ld; e += DP_THREADS) {
                const int slot = c.tok_slot[e / ld];
                c.table[e] = slot < 0 ? -1 : ops[i].table[(size_t)slot * ld + e % ld];
            }
            if (tid == 0) { c.table_of = ops[i].table; c.table_ld = ld; }
        }
        break;
    }
    __syncthreads();
    if (tid >= DP_CONSUMERS) {
        produce(c, ops, n_ops);
    } else {
        for (int i = 0; i < n_ops; ++i) {
            const DecodeOp& op = c.op[i & 1];
            // the next operation's record, asked for now, put down when this operation is done
            uint32_t next_word = 0;
            const bool fetch = i + 1 < n_ops && tid >= 32 && tid < 32 + (int)(sizeof(DecodeOp) / 4);
            if (fetch) next_word = __ldg(reinterpret_cast<const uint32_t*>(ops + i + 1) + tid - 32);
            stamp(c, i, 0);
            if (op.kind == DP_EMBED) run_embed(c, op, i);
            else if (op.kind == DP_GEMV) run_gemv(c, op, i);
            else run_attention(c, op, i);
            if (fetch) reinterpret_cast<uint32_t*>(&c.op[(i + 1) & 1])[tid - 32] = next_word;
            consumer_sync();
        }
        stamp(c, n_ops, 0);
    }
    __syncthreads();
    // the last CTA to leave counts the launch (the flags of the next one differ from all of this one's)
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(sync_words + 1, 1u);
        if (old == gridDim.x - 1) {
            sync_words[0] += 1u;
            sync_words[2] = 0u;
            __threadfence();
            sync_words[1] = 0u;
        }
    }
}

constexpr size_t DP_SMEM_BYTES = (size_t)DP_SLOTS * DP_SLOT_BYTES + DP_STAGE_BYTES + DP_RED_FLOATS * 4 + DP_TABLE_INTS * 4 + sizeof(Shared);
static_assert(DP_SMEM_BYTES <= 232448, "the decode program's shared memory exceeds what a CTA may have");
static_assert(DP_CONSUMER_WARPS * (DP_MAX_DH + 2) * 4 + 4 * DP_MAX_DH * 4 <= DP_STAGE_BYTES, "attention's merge buffers live in the staging area");
static_assert(DP_BIAS_BYTES >= 24 * 4 && sizeof(DecodeOp) / 4 <= 96, "an operation record is fetched by three warps at most");

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
int log2_exact(int v) {
    int l = 0;
    while ((1 << l) < v) ++l;
    return (1 << l) == v ? l : -1;
}
// a buffer argument: plain (fmt 0/1, ld elements) or flagged (fmt 2/3, ld groups a row, segments of `seg` columns)
bool fill_buf(Buf* b, void* p, int fmt, int ld, int seg, int dep, int cols) {
    if (p == nullptr || !aligned16(p) || fmt < FMT_F32 || fmt > FMT_LL_BF16 || ld <= 0) return false;
    b->p = p; b->fmt = fmt; b->ld = ld; b->dep = dep; b->pad = 0;
    if (dp_is_ll(fmt)) {
        const int per = dp_per(fmt);
        if (seg <= 0) seg = cols;
        b->seg = seg;
        b->gps = ((seg + per - 1) / per + 1) & ~1;
        const int n_seg = (cols + seg - 1) / seg;
        if (ld < n_seg * b->gps || ld % 2 != 0) return false;
    } else {
        b->seg = cols; b->gps = 0;
        if (ld < cols) return false;
    }
    return true;
}

}  // namespace

extern "C" int vlrf_decode_program_op_bytes() { return (int)sizeof(DecodeOp); }
extern "C" int vlrf_decode_program_max_rows() { return DP_MAX_ROWS; }

// Whether a product of these sizes and buffer formats (0 float32, 1 bfloat16, 2 flagged float32, 3 flagged bfloat16)
// is taken.  K a multiple of 32; a float32 input at most 1,984 columns wide; a norm needs a float32 input.
extern "C" int vlrf_decode_program_gemv_takes(int n_rows, int N, int K, int in_fmt, int out_fmt, int norm) {
    DecodeOp op = {};
    if (!dp_plan_gemv(n_rows, N, K, in_fmt, out_fmt, &op)) return 0;
    if (norm != DP_NORM_NONE && !(in_fmt == FMT_F32 || in_fmt == FMT_LL_F32)) return 0;
    return 1;
}

extern "C" int vlrf_decode_program_attention_takes(int head_dim, int block_tokens) {
    return log2_exact(head_dim) >= 4 && head_dim <= DP_MAX_DH && log2_exact(block_tokens) >= 5 ? 1 : 0;
}

extern "C" int vlrf_decode_op_embed(void* ops_host, int index, const void* wte, const void* wpe, const int* tokens, void* x,
                                    int x_fmt, int x_ld, int d, int V, int P) {
    VLRF_REQUIRE(ops_host != nullptr && index >= 0 && wte != nullptr && tokens != nullptr && x != nullptr, "decode program: null argument");
    VLRF_REQUIRE(d > 0 && V > 0 && (x_fmt == FMT_F32 || x_fmt == FMT_LL_F32), "decode program: an embedding writes float32 rows");
    DecodeOp op = {};
    op.kind = DP_EMBED;
    op.N = d; op.vocab = V; op.n_pos = P;
    op.W = wte; op.wpe = wpe; op.tokens = tokens;
    VLRF_REQUIRE(fill_buf(&op.out, x, x_fmt, x_ld, 0, index, d), "decode program: the embedding's output buffer does not fit");
    static_cast<DecodeOp*>(ops_host)[index] = op;
    return VLRF_OK;
}

extern "C" int vlrf_decode_op_gemv(void* ops_host, int index, int n_rows, const void* in, int in_fmt, int in_ld, int in_seg,
                                   int in_dep, int norm, const float* gamma, const float* beta, float eps, const void* W,
                                   const float* bias, int N, int K, int act, void* out, int out_fmt, int out_ld,
                                   const void* residual, int res_fmt, int res_ld, int res_dep, void* kc, void* vc,
                                   const int* block_table, int max_blocks, int k_off, int v_off, int Hkv, int dh, int BT) {
    VLRF_REQUIRE(ops_host != nullptr && index >= 0 && in != nullptr && W != nullptr && out != nullptr, "decode program: null argument");
    DecodeOp op = {};
    op.kind = DP_GEMV;
    VLRF_REQUIRE(dp_plan_gemv(n_rows, N, K, in_fmt, out_fmt, &op) && vlrf_decode_program_gemv_takes(n_rows, N, K, in_fmt, out_fmt, norm),
                 "decode program: a product of %d rows, N=%d, K=%d (formats %d to %d, norm %d) is not taken: K a multiple of 32, at "
                 "most %d rows, a float32 input at most %d columns wide", n_rows, N, K, in_fmt, out_fmt, norm, DP_MAX_ROWS, DP_MAX_K_F32);
    VLRF_REQUIRE(aligned16(W) && aligned16(bias), "decode program: weights must be 16-byte aligned");
    VLRF_REQUIRE(norm == DP_NORM_NONE || (gamma != nullptr && aligned16(gamma) && (beta == nullptr || aligned16(beta))),
                 "decode program: a norm needs its weight");
    op.N = N; op.K = K; op.norm = norm; op.act = act; op.eps = eps;
    op.gamma = gamma; op.beta = beta; op.W = W; op.bias = bias;
    VLRF_REQUIRE(fill_buf(&op.in, const_cast<void*>(in), in_fmt, in_ld, in_seg, in_dep, K) && (in_fmt != FMT_BF16 || in_ld % 8 == 0) &&
                 (in_fmt != FMT_F32 || in_ld % 4 == 0), "decode program: the input buffer does not fit");
    VLRF_REQUIRE(fill_buf(&op.out, out, out_fmt, out_ld, 0, index, N), "decode program: the output buffer does not fit");
    if (residual != nullptr) {
        VLRF_REQUIRE((out_fmt == FMT_F32 && res_fmt == FMT_F32) || (out_fmt == FMT_LL_F32 && res_fmt == FMT_LL_F32),
                     "decode program: a residual is float32, in the format of the output");
        VLRF_REQUIRE(fill_buf(&op.res, const_cast<void*>(residual), res_fmt, res_ld, 0, res_dep, N), "decode program: the residual buffer does not fit");
    }
    if (kc != nullptr) {
        VLRF_REQUIRE((out_fmt == FMT_BF16 || out_fmt == FMT_LL_BF16) && vc != nullptr && block_table != nullptr && Hkv > 0 &&
                     log2_exact(dh) >= 0 && log2_exact(BT) >= 0 && k_off >= 0 && v_off >= 0 && k_off + Hkv * dh <= N && v_off + Hkv * dh <= N,
                     "decode program: the cache scatter does not match the projection (head size and block size powers of two)");
        op.kc = kc; op.vc = vc; op.table = block_table; op.table_ld = max_blocks;
        op.k_off = k_off; op.v_off = v_off; op.hkv = Hkv; op.dh = dh; op.bt = BT;
        op.log2_dh = log2_exact(dh); op.log2_bt = log2_exact(BT);
    }
    static_cast<DecodeOp*>(ops_host)[index] = op;
    return VLRF_OK;
}

extern "C" int vlrf_decode_op_attention(void* ops_host, int index, const void* qkv, int qkv_fmt, int qkv_ld, int qkv_dep,
                                        int qkv_cols, int q_off, int k_off, int v_off, const void* kc, const void* vc,
                                        const int* block_table, int max_blocks, void* out, int out_fmt, int out_ld, int H,
                                        int Hkv, int dh, int BT, float scale, int window, int n_split, float* partials,
                                        int* counters) {
    VLRF_REQUIRE(ops_host != nullptr && index >= 0 && qkv != nullptr && kc != nullptr && vc != nullptr && block_table != nullptr &&
                 out != nullptr, "decode program: null argument");
    VLRF_REQUIRE(vlrf_decode_program_attention_takes(dh, BT), "decode program: attention with head size %d is not taken (16, 32, 64, 128, 256)", dh);
    VLRF_REQUIRE(H > 0 && Hkv > 0 && H % Hkv == 0 && n_split >= 1, "decode program: heads do not match");
    VLRF_REQUIRE(n_split == 1 || (partials != nullptr && counters != nullptr), "decode program: parts need scratch");
    VLRF_REQUIRE((qkv_fmt == FMT_BF16 || qkv_fmt == FMT_LL_BF16) && (out_fmt == FMT_BF16 || out_fmt == FMT_LL_BF16),
                 "decode program: attention reads and writes bfloat16 rows");
    VLRF_REQUIRE(aligned16(kc) && aligned16(vc) && q_off >= 0 && q_off + H * dh <= qkv_cols, "decode program: attention operands");
    VLRF_REQUIRE(qkv_fmt == FMT_BF16 || (k_off >= 0 && v_off >= 0 && k_off + Hkv * dh <= qkv_cols && v_off + Hkv * dh <= qkv_cols),
                 "decode program: a flagged q/k/v buffer also holds the newest key and value");
    DecodeOp op = {};
    op.kind = DP_ATTENTION;
    op.q_off = q_off; op.k_off = k_off; op.v_off = v_off; op.kc = const_cast<void*>(kc); op.vc = const_cast<void*>(vc);
    op.table = block_table; op.table_ld = max_blocks;
    op.n_heads = H; op.hkv = Hkv; op.dh = dh; op.bt = BT; op.scale = scale; op.window = window; op.n_split = n_split;
    op.log2_dh = log2_exact(dh); op.log2_bt = log2_exact(BT);
    op.partials = partials; op.counters = counters;
    VLRF_REQUIRE(fill_buf(&op.in, const_cast<void*>(qkv), qkv_fmt, qkv_ld, 0, qkv_dep, qkv_cols), "decode program: the q/k/v buffer does not fit");
    VLRF_REQUIRE(fill_buf(&op.out, out, out_fmt, out_ld, dh, index, H * dh), "decode program: the output buffer does not fit");
    static_cast<DecodeOp*>(ops_host)[index] = op;
    return VLRF_OK;
}

// Runs the operations (device array of vlrf_decode_program_op_bytes() each, filled on the host by the functions
// above and copied over) for n_rows rows whose slots and positions are tok_slot / tok_pos.  sync_words: 4 uint32
// on the device, zero before the first launch; [0] counts the launches (the flags of flagged buffers are made from
// it, so such buffers belong to one sync_words).  One launch; launches that share sync_words, or buffers named in the
// operations, must not overlap.  trace: null, or int64 [CTAs = SMs][n_ops + 1][8] on the device that receives
// times in nanoseconds: [cta][op][0] the CTA begins the operation ([cta][n_ops][0]: it has finished the last),
// [cta][op][1…4] stages inside it (zero where the CTA had no share of the operation).
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
