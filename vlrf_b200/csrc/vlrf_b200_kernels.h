// The C interface of libvlrf_b200_kernels.so: every kernel of the library as a plain C function, for callers
// that drive the kernels without Python (the Python package calls exactly these through ctypes).
//
// Conventions, the same for every function (status codes in the manner of the reference's include/api/vlrf.h:32-41):
//   * Pointers are device pointers unless a comment says otherwise; matrices are row-major and contiguous, `ld*` is
//     the distance between rows in elements.  `dtype` arguments are VLRF_F32 or VLRF_BF16.
//   * A function checks its sizes on the host, launches on `stream`, and returns VLRF_OK or a status whose text
//     vlrf_last_error() gives (per thread).  A size that a kernel does not take is refused, never computed wrongly;
//     the *_takes functions say beforehand whether a kernel takes a shape.
//   * Nothing allocates device memory.  Scratch comes from the caller (vlrf_attn_decode_noalloc, declared in
//     attention_decode_noalloc.h, is the one exception: its scratch lies in the library's image).
//   * `dev_err` is one int32 on the device that kernels OR bits into (VLRF_DEVERR_*) instead of faulting: a token id
//     or position out of range is clamped, a token whose cache block is not mapped is skipped, a bounded wait that
//     ran out is recorded.  The caller reads and clears it when it likes.
//   * Kernels are launched with programmatic stream serialization unless vlrf_set_chained_launch(0) was called: a
//     kernel may begin while the one before it on the stream still runs, and waits inside for its completion before
//     it touches what that kernel writes.
//   * The paged cache: K and V of one layer are [n_blocks][Hkv][BT][dh]; block_table is int32 [slots][max_blocks],
//     entry (s, i) the block that holds tokens i·BT … of slot s, or −1; BT is 64 in this library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VLRF_OK 0
#define VLRF_ERR_INVALID_ARG 1
#define VLRF_ERR_UNSUPPORTED 2
#define VLRF_ERR_CUDA 3

#define VLRF_F32 0
#define VLRF_BF16 1

#define VLRF_ACT_NONE 0
#define VLRF_ACT_GELU_TANH 1
#define VLRF_ACT_GELU_ERF 2

#define VLRF_DEVERR_TOKEN_RANGE 1
#define VLRF_DEVERR_POSITION_RANGE 2
#define VLRF_DEVERR_NO_BLOCK 4
#define VLRF_DEVERR_WAIT_TIMEOUT 8

// ---- status -------------------------------------------------------------------------------------------------
// Text of the calling thread's last failure (host pointer, valid until the thread's next failure).
const char* vlrf_last_error();
// Properties of the current device (host pointers).
int vlrf_device_info(int* sm_count, int* cc_major, int* cc_minor, int* max_smem_optin);
// Whether kernels are launched chained (programmatic stream serialization); on by default.
int vlrf_chained_launch_enabled();
int vlrf_set_chained_launch(int on);
// Time stamps that the decode step's kernels leave in a build with -DVLRF_KERNEL_TRACE: the buffer's sizes (0 slots
// in a build without stamps), and a copy of it to host memory, [slots][ctas][2 + stations] int64 (launch number,
// kind of kernel: 1 few-row product, 2 decode attention, 3 many-row product, 4 prompt attention; then the global timer's nanoseconds at every station),
// after which the buffer is cleared.
long long* vlrf_trace_buffer();                 // the buffer on the device (what the kernels are handed), or null
int vlrf_trace_dims(int* slots, int* ctas, int* stations);
int vlrf_trace_read(long long* host);

// ---- embedding and LayerNorm (embed_norm.cu) ----------------------------------------------------------------
// x[t] = wte[tokens[t]] (+ wpe[positions[t]] if wpe is not null), float32 [T][d]; tables [V][d] and [P][d] of
// w_dtype.  stats (or null): per row and 32-column segment the sum and the squared deviation from the segment's
// mean, [T][ceil(d/32)][2], for a later product that norms these rows (vlrf_gemm_splitk).
int vlrf_embed(const void* wte, const void* wpe, int w_dtype, const int* tokens, const int* positions, float* x, int T,
               int d, int V, int P, float* stats, int* dev_err, cudaStream_t stream);
// out[r] = LayerNorm(x[rows ? rows[r] : r]) · gamma + beta, statistics in float32 over the whole row (two passes);
// x float32 [·][d], out of out_dtype [n_rows][d].
int vlrf_layernorm(const float* x, const int* rows, const float* gamma, const float* beta, void* out, int out_dtype,
                   int n_rows, int d, float eps, cudaStream_t stream);

// ---- products: Y[M][N] = act(X[M][K] · W[N][K]ᵀ + bias) (+ residual) ----------------------------------------------
// bias float32 [N] or null; residual float32 [M][ldy] or null (it may be Y itself); act is VLRF_ACT_*.  The
// optional cache scatter (Kc not null) also writes the K and V columns of a fused q/k/v projection (columns
// k_off … and v_off …, Hkv heads of dh) into one layer's paged cache at each row's (tok_slot, tok_pos).

// Any sizes, any dtype, FMAs only (the true 32-bit product; the sum over k runs in an order that does not depend on M).
int vlrf_gemm_simt(const void* X, const void* W, const float* bias, const float* residual, void* Y, int M, int N, int K,
                   int ldx, int ldy, int in_dtype, int out_dtype, int act, cudaStream_t stream);

// Many rows, bfloat16 X and W, on the tcgen05 tensor cores (TMA ring, accumulators in tensor memory); with few rows
// and very many columns the operands' roles are exchanged.  K a multiple of 8.
int vlrf_gemm_tcgen05_takes(int M, int N, int K, int ldx);
int vlrf_gemm_tcgen05(const void* X, const void* W, const float* bias, const float* residual, void* Y, int M, int N, int K,
                      int ldx, int ldy, int out_dtype, int act, void* Kc, void* Vc, const int* block_table,
                      int max_blocks, const int* tok_slot, const int* tok_pos, int k_off, int v_off, int Hkv, int dh,
                      int BT, int* dev_err, cudaStream_t stream);
// For measurements: force the tile width (64 … 256 in steps of 32), 0 = chosen by size again.
int vlrf_gemm_tcgen05_force_width(int bn);

// Few rows (M ≤ 64), the sum over k cut into parts whose CTAs form a cluster and add through distributed shared
// memory.  x_is_f32_ln: X is the float32 residual stream and LayerNorm (gamma, beta, eps) is applied first, from
// the rows' statistics `stats_in` ([M][ceil(K/32)][2], see vlrf_embed; M ≤ 16).  stats_out (or null): the same
// statistics of the float32 rows of Y.
long long vlrf_row_stats_floats(int rows, int width);
int vlrf_gemm_splitk_takes(int M, int N, int K, int ldx, int x_is_f32_ln);
int vlrf_gemm_splitk(const void* X, int x_is_f32_ln, const void* W, const float* bias, const float* residual, void* Y,
                     int out_dtype, int M, int N, int K, int ldx, int ldy, int act, const float* gamma, const float* beta,
                     float eps, void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                     const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT, const float* stats_in,
                     float* stats_out, int* dev_err, cudaStream_t stream);

// Few rows, weights streamed once through persistent CTAs (`mma.sync`); x_is_f32_ln: the norm of whole rows in
// the prologue (vlrf_gemm_skinny_ln_fits says whether M rows of K columns fit).  sm_count: CTAs to launch.
int vlrf_gemm_skinny_ln_fits(int M, int K);
int vlrf_gemm_skinny(const void* X, int x_is_f32_ln, const void* W, const float* bias, const float* residual, void* Y,
                     int out_dtype, int M, int N, int K, int ldx, int ldy, int act, const float* gamma, const float* beta,
                     float eps, void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                     const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT, int sm_count, int* dev_err,
                     cudaStream_t stream);

// ---- attention over the paged cache ------------------------------------------------------------------------------
// Rows of `qkv` hold a token's fused projection (row stride ld); queries start at column q_off, H heads of dh; Hkv
// key/value heads (H a multiple of Hkv).  A key at position k is visible to the query at position p iff k ≤ p and,
// with window > 0, p − k < window.  Scores are scaled by `scale`; softmax, sums and outputs in float32.  `out` is
// [rows][ld_out] of the dtype of qkv.

// The new tokens' K and V columns into the cache (where no product's epilogue has written them).
int vlrf_kv_append(const void* qkv, int dtype, int ld, int k_off, int v_off, void* Kc, void* Vc, const int* block_table,
                   int max_blocks, const int* tok_slot, const int* tok_pos, int T, int Hkv, int dh, int BT, int* dev_err,
                   cudaStream_t stream);
// Any mix of tokens, any head size that is a multiple of 16, float32 or bfloat16: a warp per (token, head).
int vlrf_attn_generic(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc,
                      const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos, void* out,
                      int ld_out, int T, int H, int Hkv, int dh, int BT, float scale, int window, int* dev_err,
                      cudaStream_t stream);

// A prompt step in bfloat16: sequence i brings the rows seq_start[i] … seq_start[i+1]−1, which continue slot
// seq_slot[i] at position seq_pos0[i]; max_new is the longest run.  n_blocks: blocks of the cache.
// `mma.sync` kernel, head sizes 64 and 128:
int vlrf_attn_prefill_takes(int dh, int BT, int ld, int q_off);
int vlrf_attn_prefill(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                      const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                      const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new, int H, int Hkv,
                      int dh, int BT, float scale, int window, int* dev_err, cudaStream_t stream);
// tcgen05 kernel, head size 64.  With n_parts > 1 the keys of a long tile of queries are dealt to up to n_parts
// CTAs that meet in scratch: partials, float32, (tiles · n_parts · vlrf_attn_prefill_tc_part_floats()) with tiles =
// ceil(max_new / vlrf_attn_prefill_tc_tile()) · n_seqs · H; counters, int32 [tiles], zero before the first call
// (every call leaves them zero).
int vlrf_attn_prefill_tc_takes(int dh, int BT, int ld, int q_off, int ld_out);
int vlrf_attn_prefill_tc_part_floats();
int vlrf_attn_prefill_tc_max_parts();
int vlrf_attn_prefill_tc_min_part_blocks();
int vlrf_attn_prefill_tc_tile();
int vlrf_attn_prefill_tc(const void* qkv, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                         const int* block_table, int max_blocks, const int* seq_slot, const int* seq_start,
                         const int* seq_pos0, void* out, int ld_out, int n_tokens, int n_seqs, int max_new, int H,
                         int Hkv, int dh, int BT, float scale, int window, int n_parts, float* partials, int* counters,
                         int* dev_err, cudaStream_t stream);

// A decode step: one query per row, at position tok_pos[row] of slot tok_slot[row] (−1: padding, skipped); each
// context is cut into n_split parts, one CTA each.  Head sizes 64 and 128 with up to 16 parts merge inside a
// thread-block cluster and need no scratch (vlrf_attn_decode_needs_scratch says); otherwise partials, float32
// (vlrf_attn_decode_scratch_floats), and counters, int32 [rows · H], zero between calls.  n_blocks: blocks of the
// cache, or 0 if unknown (then bfloat16 with head size 64 takes the kernel without tensor maps).
int vlrf_attn_decode_needs_scratch(int dh, int n_split);
long long vlrf_attn_decode_scratch_floats(int rows, int H, int dh, int n_split);
int vlrf_attn_decode(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc, int n_blocks,
                     const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos, void* out,
                     int ld_out, int rows, int H, int Hkv, int dh, int BT, float scale, int window, int n_split,
                     float* partials, int* counters, int* dev_err, cudaStream_t stream);
// The same for callers that cannot allocate scratch: see attention_decode_noalloc.h for its rules and limits.
int vlrf_attn_decode_noalloc(const void* qkv, int dtype, int ld, int q_off, const void* Kc, const void* Vc,
                             const int* block_table, int max_blocks, const int* tok_slot, const int* tok_pos, void* out,
                             int ld_out, int rows, int H, int Hkv, int dh, int BT, float scale, int window, int n_split,
                             int* dev_err, cudaStream_t stream);

// ---- sampling (sampling.cu) ----------------------------------------------------------------------------------------
// One token per row of float32 logits [n_rows][ld] over V entries, in the order of the reference (include/model/
// transformer.hpp:124-182): temperature[r] ≤ 0 → the first maximum; else softmax(logits / temperature), top_k[r]
// (≤ 0: off), top_p[r] (≥ 1: off), and an inverse-CDF draw from the counter-based stream (rng_key[r], rng_ctr[r]),
// whose counter moves on.  temperature null: every row greedy; top_k or top_p null: off; rows that draw need rng_key
// and rng_ctr.  next_token,
// next_pos, row_slot (or null): the chosen token goes into next_token[r] as well and next_pos[r] grows by one for
// rows with row_slot[r] ≥ 0, so that the next decode step needs nothing from the host.
int vlrf_sample(const float* logits, int ld, int n_rows, int V, const float* temperature, const int* top_k,
                const float* top_p, const unsigned long long* rng_key, unsigned int* rng_ctr, int* out_token,
                int* next_token, int* next_pos, const int* row_slot, cudaStream_t stream);
// Repetition, frequency and presence penalties over the tokens generated so far (gen [n_rows][gen_ld], gen_len)
// and the no-repeat n-gram block (ngram[r] ≤ 0: off), on the raw logits, in place (reference :124-141).
int vlrf_apply_penalties(float* logits, int ld, int n_rows, int V, const int* gen, int gen_ld, const int* gen_len,
                         const float* rep, const float* freq, const float* pres, const int* ngram, cudaStream_t stream);

// ---- a whole decode step as one persistent kernel (decode_program.cu) ----------------------------------------
// The step is a list of operations (embedding; few-row product with an optional norm of its input, bias, activation,
// residual and cache scatter; attention of one query per row and head over the paged cache), filled on the HOST one
// record at a time by the vlrf_decode_op_* functions into an array of vlrf_decode_program_op_bytes() bytes a record,
// copied to the device by the caller, and run by vlrf_decode_program_run: one cooperative launch of one CTA per SM.
// At most vlrf_decode_program_max_rows() rows; bfloat16 weights and caches.  norm: 0 none, 1 LayerNorm (beta may be
// null), 2 RMS norm.  Buffers between operations have a format: 0 float32 rows, 1 bfloat16 rows (`ld` elements a
// row), or flagged rows, 2: groups of 16 bytes holding 3 float32 and a flag, 3: 6 bfloat16 and a flag (`ld` groups a
// row; `seg` > 0 cuts a row's columns into segments that each begin a new group; zero-filled before first use).
// An operation that reads a flagged buffer waits, group by group, for the flag of the operation `dep` (its index in
// the list) that writes it in the same launch; there is no other ordering between operations, so plain buffers must
// be complete before the launch, and a flagged buffer may be rewritten only by an operation that cannot begin before
// every reader of the old contents has finished.  The *_takes functions say whether an operation's sizes are taken.
int vlrf_decode_program_op_bytes();
int vlrf_decode_program_max_rows();
int vlrf_decode_program_gemv_takes(int n_rows, int N, int K, int in_fmt, int out_fmt, int norm);
int vlrf_decode_program_attention_takes(int head_dim, int block_tokens);
int vlrf_decode_op_embed(void* ops_host, int index, const void* wte, const void* wpe, const int* tokens, void* x, int x_fmt,
                         int x_ld, int d, int V, int P);
int vlrf_decode_op_gemv(void* ops_host, int index, int n_rows, const void* in, int in_fmt, int in_ld, int in_seg, int in_dep,
                        int norm, const float* gamma, const float* beta, float eps, const void* W, const float* bias, int N,
                        int K, int act, void* out, int out_fmt, int out_ld, const void* residual, int res_fmt, int res_ld,
                        int res_dep, void* kc, void* vc, const int* block_table, int max_blocks, int k_off, int v_off, int Hkv,
                        int dh, int BT);
// With a flagged q/k/v buffer the newest key and value are read from it (columns k_off, v_off) and the cache up to the
// position before; with a plain one the cache holds every key.  A flagged output has one segment a head.
int vlrf_decode_op_attention(void* ops_host, int index, const void* qkv, int qkv_fmt, int qkv_ld, int qkv_dep, int qkv_cols,
                             int q_off, int k_off, int v_off, const void* kc, const void* vc, const int* block_table,
                             int max_blocks, void* out, int out_fmt, int out_ld, int H, int Hkv, int dh, int BT, float scale,
                             int window, int n_split, float* partials, int* counters);
// sync_words: 4 uint32 on the device, zero before the first launch; [0] counts the launches (flags are made from it, so
// flagged buffers belong to one sync_words).  Launches that share them, or buffers that the operations name, must not
// overlap.  trace: null, or int64 [SMs][n_ops + 1][8] on the device: times (ns), [cta][op][0] the CTA begins the
// operation ([cta][n_ops][0]: it has finished the last), [cta][op][1…4] stages inside it (0: no share of it).
int vlrf_decode_program_run(const void* ops_dev, int n_ops, int n_rows, const int* tok_slot, const int* tok_pos,
                            void* sync_words, int* dev_err, long long* trace, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
