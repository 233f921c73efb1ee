// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (VLRF-org/VLRF has no GPU allocator to avoid and no
// split-context attention); it exists for users of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits — inside a real-time or latency-critical
// loop that must not take the allocator's locks, in a host process whose memory plan is fixed up front, or
// a plugin that is handed inputs and outputs but no allocator.  The
// ordinary entry point, vlrf_attn_decode, needs scratch memory from its caller when a context is cut into
// several parts (partial results of the parts, and a counter per (row, head)); such callers have nowhere
// to get it from.  Here the scratch is a fixed array inside the library itself, so the caller passes only
// inputs and outputs.
//
// Limits and rules:
//   * rows · heads                          ≤ VLRF_NOALLOC_MAX_ROW_HEADS        (2,048)
//   * rows · heads · n_split · (head_dim+2) ≤ VLRF_NOALLOC_MAX_PARTIAL_FLOATS   (2,162,688 floats ≈ 8.3 MiB)
//     e.g. 64 rows × 32 heads × 8 splits at head size 128, or 64 × 25 × 16 at head size 64.
//     Larger sizes are refused with an error that names the limit; nothing is launched then.
//   * Every GPU that loads the library holds these ≈ 8.3 MiB until the process ends.
//   * The first call on a device looks up the arrays' device addresses (cudaGetSymbolAddress) with that
//     device current.  Make that first call outside of any stream capture.
//   * All calls on a device share the one scratch array, and it keeps what the last call left.  The
//     counters are cleared at the start of every call (a cudaMemsetAsync on the given stream); the
//     partials are always written before they are read.  Two calls that overlap on the GPU (different
//     streams, no ordering between them) race on the scratch and give wrong results: order them.
//   * Nothing is allocated or freed: no cudaMalloc, no cudaFree, no library routine that allocates.
//
// Arguments are those of vlrf_attn_decode without `n_blocks`, `partials` and `counters`; returns 0 or a
// status whose text vlrf_last_error() gives.  Without the pool's block count no tensor map of the cache can
// be made, so bfloat16 with head size 64 runs here on the kernel that copies keys and values in bulk and
// multiplies on the CUDA cores, not on the `mma.sync` kernel that vlrf_attn_decode picks for those sizes:
// the same sums in another order, equal within rounding, and slower.
#pragma once
#include <cuda_runtime.h>

#define VLRF_NOALLOC_MAX_ROW_HEADS 2048
#define VLRF_NOALLOC_MAX_PARTIAL_FLOATS (2048 * 8 * 132)

extern "C" int vlrf_attn_decode_noalloc(const void* qkv, int dtype, int ld, int q_off, const void* Kc,
                                        const void* Vc, const int* block_table, int max_blocks,
                                        const int* tok_slot, const int* tok_pos, void* out, int ld_out,
                                        int rows, int H, int Hkv, int dh, int BT, float scale, int window,
                                        int n_split, int* dev_err, cudaStream_t stream);
