// Y[M,N] = act(X[M,K] · W[N,K]^T + bias) (+ residual) for few rows (M ≤ 64): the decode step's products.
//
// With a handful of rows the product is bound by reading W once, and an SM's load/store unit cannot keep
// enough ordinary loads in flight to cover HBM's latency.  So W is moved by TMA: a persistent CTA takes
// groups of 8·CG rows of W (its output columns) and requests each group's slab as tiled tensor loads
// (`cp.async.bulk.tensor.2d`, boxes of 64 k × 8·CG rows, 128-byte swizzle, out-of-range rows read as
// zeros) into a ring of up to four shared-memory stages, each segment of a slab completing on its own
// mbarrier; the slab of group i+S is requested as soon as every warp has finished with group i, so the
// weight stream of an SM does not stop while it has groups left.  The input rows are staged once per CTA,
// either by TMA or by the fused LayerNorm, in the same swizzled layout.  Eight warps take the 32-wide
// k-chunks in turn as the segments land: the batch rows are the 16-row operand of
// `mma.sync.m16n8k16` (bf16 in, float32 accumulate), 8 rows of W the 8-column operand; since a sum over k
// may run in any order, the 8 values of one 16-byte shared-memory read feed two MMAs directly, and the
// swizzle makes those reads conflict-free.  Warps that share output columns add their partial sums in a
// fixed order.  Waits on the mbarriers are bounded: a wait that gives up sets a bit in the device error
// word and the CTA writes nothing more.
//
// The kernel is launched so that it may begin while the kernel before it still runs: it requests its
// first weight slabs, then waits for that kernel, then touches the activations.
//
// Fusions: LayerNorm of the float32 residual rows in the prologue (statistics in float32, two passes over
// registers; reference include/model/ops.hpp:443-476), bias / GELU / residual sum in the epilogue (reference
// include/model/feedforward.hpp:54-76, include/model/transformer_block.hpp:153,158), and the scatter of
// the K and V columns of a fused q/k/v projection into the paged cache (reference
// include/model/kv_cache.hpp:215-251).
#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int SK_THREADS = 512;
constexpr int SK_WARPS = 16;
constexpr int MAX_SEG = 8;
constexpr int MAX_STAGES = 4;
constexpr uint32_t WAIT_LIMIT = 4000000u;   // polls of a barrier before giving up (far beyond any real wait)

struct KvScatter {
    void* Kc; void* Vc;            // this layer's cache [block][kv_head][BT][dh], bf16
    const int* block_table; const int* tok_slot; const int* tok_pos;
    int max_blocks, k_off, v_off, width, dh, Hkv, BT;   // width = Hkv*dh
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// k is cut into tiles of 64 (128 bytes a row); tiles are grouped into at most MAX_SEG segments
struct Tiling { int n_tiles, tiles_per_seg, n_seg; };
__host__ __device__ __forceinline__ Tiling tiling(int K) {
    const int n_tiles = (K + 63) / 64;
    const int tps = (n_tiles + MAX_SEG - 1) / MAX_SEG;
    return Tiling{n_tiles, tps, (n_tiles + tps - 1) / tps};
}
// byte offset of the 16-byte piece `piece` (0…7) of row `row` inside a swizzled tile of 128-byte rows
__device__ __forceinline__ int swz(int row, int piece) { return row * 128 + ((piece ^ (row & 7)) << 4); }

// XMODE 0: X bf16 read from global per fragment; 1: X bf16 staged in shared memory by TMA;
//       2: X float32, LayerNorm applied, result staged as bf16
template <int MT16, int XMODE, typename OT>
__global__ void __launch_bounds__(SK_THREADS)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const void* __restrict__ Xv, const float* __restrict__ bias, const float* residual, OT* Y,
                   int M, int N, int K, int ldx, int ldy, int act, int CG, int S,
                   const float* __restrict__ gamma, const float* __restrict__ beta, float eps, KvScatter kv,
                   int* __restrict__ dev_err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    // The MMA fixes which lane holds which row of a fragment, but not which row of the tile that is: fragment
    // row g is tile row pg = g/2 + 4·(g mod 2).  Then the eight lanes that read shared memory together
    // (two fragment rows × four 16-byte pieces) touch tile rows that differ in bit 2, and under the
    // 128-byte swizzle their pieces fall into eight different bank groups.  Fragment column c of the
    // result is tile row π(c) of W in the same way: columns 2t and 2t+1 are rows t and t+4.
    const int pg = (g >> 1) | ((g & 1) << 2);
    const int rows_w = 8 * CG;
    constexpr int XR = 16 * MT16;                      // rows of the staged X tile
    const Tiling tl = tiling(K);
    const int n_groups = (N + rows_w - 1) / rows_w;
    const int n_my = ((int)blockIdx.x < n_groups) ? (n_groups - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    const size_t tile_bytes = (size_t)rows_w * 128;
    const size_t stage_bytes = tile_bytes * tl.n_tiles;
    unsigned char* ws = smem;                                                  // [S][n_tiles][rows_w][128]
    unsigned char* xs = ws + (size_t)S * stage_bytes;                          // [n_tiles][XR][128] (XMODE 1, 2)
    float* red = reinterpret_cast<float*>(xs + (XMODE != 0 ? (size_t)tl.n_tiles * XR * 128 : 0));   // [2][warps][MT16*128]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + 2 * SK_WARPS * MT16 * 4 * 32);              // [S][MAX_SEG]

    if (threadIdx.x == 0) {
        tma_prefetch_descriptor(&tmap_w);
        if (XMODE == 1) tma_prefetch_descriptor(&tmap_x);
        for (int i = 0; i < S * MAX_SEG; ++i) mbar_init(&bars[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // Lane sgi of warp 0 requests segment sgi of a slab: it announces the bytes on the segment's barrier
    // and issues one tiled load per 64-wide k tile.  `with_x`: the request also brings the X rows.
    auto request = [&](int it, bool with_x) {
        if (lane >= tl.n_seg) return;
        const int stage = it % S;
        const int n_base = ((int)blockIdx.x + it * (int)gridDim.x) * rows_w;
        const int t0 = lane * tl.tiles_per_seg, t1 = min(tl.n_tiles, t0 + tl.tiles_per_seg);
        uint64_t* bar = &bars[stage * MAX_SEG + lane];
        mbar_expect_tx(bar, (uint32_t)((t1 - t0) * (tile_bytes + (with_x ? (size_t)XR * 128 : 0))));
        for (int tile = t0; tile < t1; ++tile) {
            tma_load_2d(ws + (size_t)stage * stage_bytes + (size_t)tile * tile_bytes, &tmap_w, tile * 64, n_base, bar);
            if (with_x) tma_load_2d(xs + (size_t)tile * XR * 128, &tmap_x, tile * 64, 0, bar);
        }
    };

    // weights do not depend on the kernel before this one: the first slabs are requested at once
    // (when X comes by TMA too, the first slab's request waits for it; the others go now)
    if (warp == 0)
        for (int it = (XMODE == 1 ? 1 : 0); it < min(S, n_my); ++it) request(it, false);
    pdl_launch_dependents();      // the next kernel may start fetching its weights behind ours
    pdl_wait();                   // from here on the rows that the kernel before wrote may be read
    if (XMODE == 1 && warp == 0 && n_my > 0) request(0, true);

    if (XMODE == 2) {
        const float* X = reinterpret_cast<const float*>(Xv);
        const bool cached = (K % 128 == 0) && K <= 1024 && (ldx % 4 == 0);
        for (int m = warp; m < M; m += SK_WARPS) {
            const float* row = X + (size_t)m * ldx;
            // element k of row m sits in tile k/64 at the swizzled place of its 16-byte piece
            auto place = [&](int k) -> __nv_bfloat16* {
                return reinterpret_cast<__nv_bfloat16*>(xs + (size_t)(k >> 6) * XR * 128 + swz(m, (k & 63) >> 3)) + (k & 7);
            };
            if (cached) {
                // the row is read once, 16 bytes a lane a load, and stays in registers for both passes
                float4 v[8];
                const int nv = K / 128;
                float s = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < nv) {
                        v[j] = *reinterpret_cast<const float4*>(row + (j * 32 + lane) * 4);
                        s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
                    }
                const float mean = warp_sum(s) / (float)K;
                float q = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < nv) {
                        const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, d = v[j].w - mean;
                        q += (a * a + b * b) + (c * c + d * d);
                    }
                const float inv = 1.f / sqrtf(warp_sum(q) / (float)K + eps);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (j < nv) {
                        const int i = (j * 32 + lane) * 4;
                        const float4 gm = *reinterpret_cast<const float4*>(gamma + i);
                        const float4 bt = *reinterpret_cast<const float4*>(beta + i);
                        __nv_bfloat16* dst = place(i);
                        *reinterpret_cast<__nv_bfloat162*>(dst) =
                            __floats2bfloat162_rn((v[j].x - mean) * inv * gm.x + bt.x, (v[j].y - mean) * inv * gm.y + bt.y);
                        *reinterpret_cast<__nv_bfloat162*>(dst + 2) =
                            __floats2bfloat162_rn((v[j].z - mean) * inv * gm.z + bt.z, (v[j].w - mean) * inv * gm.w + bt.w);
                    }
                continue;
            }
            float s = 0.f;
            for (int i = lane; i < K; i += 32) s += row[i];
            const float mean = warp_sum(s) / (float)K;
            float q = 0.f;
            for (int i = lane; i < K; i += 32) { const float c = row[i] - mean; q += c * c; }
            const float inv = 1.f / sqrtf(warp_sum(q) / (float)K + eps);
            for (int i = lane; i < K; i += 32)
                *place(i) = __float2bfloat16_rn((row[i] - mean) * inv * gamma[i] + beta[i]);
        }
        __syncthreads();
    }

    const int wpg = SK_WARPS / CG;                     // warps that share an 8-column group
    const int sub = warp / wpg, kpart = warp % wpg;
    const __nv_bfloat16* Xb = reinterpret_cast<const __nv_bfloat16*>(Xv);
    bool gave_up = false;

    // the rows' cache coordinates for the K/V scatter do not change from group to group
    int kv_blk[MT16][2], kv_off[MT16][2];
    if (kv.Kc != nullptr && kpart == 0) {
#pragma unroll
        for (int mt = 0; mt < MT16; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int m = mt * 16 + pg + hh * 8;
                kv_blk[mt][hh] = -2;                   // −2: nothing to write for this row
                kv_off[mt][hh] = 0;
                if (m < M) {
                    const int slot = kv.tok_slot[m];
                    if (slot >= 0) {
                        const int pos = kv.tok_pos[m];
                        kv_blk[mt][hh] = kv.block_table[(size_t)slot * kv.max_blocks + pos / kv.BT];
                        kv_off[mt][hh] = pos % kv.BT;
                    }
                }
            }
    }

    for (int it = 0; it < n_my; ++it) {
        const int stage = it % S;
        const uint32_t parity = (uint32_t)((it / S) & 1);
        const int n0 = ((int)blockIdx.x + it * (int)gridDim.x) * rows_w + sub * 8;
        // what the epilogue adds is fetched now, under the shadow of the weight copies
        float pre[MT16][4];
        float pre_bias[2] = {0.f, 0.f};
        if (kpart == 0) {
#pragma unroll
            for (int mt = 0; mt < MT16; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int m = mt * 16 + pg + ((j & 2) ? 8 : 0);
                    const int n = n0 + t + 4 * (j & 1);
                    pre[mt][j] = (n < N && m < M && residual) ? residual[(size_t)m * ldy + n] : 0.f;
                }
            if (bias) {
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    if (n0 + t + 4 * j < N) pre_bias[j] = bias[n0 + t + 4 * j];
            }
        }

        float acc[MT16][4];
#pragma unroll
        for (int i = 0; i < MT16; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
        // A warp takes the 64-wide k tiles kpart, kpart + wpg, … of its 8 columns.  Everything that does not
        // change from tile to tile (the swizzled places of this lane's pieces) is computed once.
        const int wrow = sub * 8 + pg;
        const unsigned char* wp = ws + (size_t)stage * stage_bytes + (size_t)kpart * tile_bytes;
        const int w_off0 = swz(wrow, t), w_off1 = swz(wrow, 4 + t);
        const unsigned char* xp = xs + (size_t)kpart * XR * 128;
        const size_t w_step = (size_t)wpg * tile_bytes, x_step = (size_t)wpg * XR * 128;
        int next_wait_tile = 0, seg = 0;               // the first tile of the next segment not yet waited for
        for (int tile = kpart; tile < tl.n_tiles; tile += wpg, wp += w_step, xp += x_step) {
            while (tile >= next_wait_tile && !gave_up) {
                uint32_t polls = 0;
                while (!mbar_try_wait(&bars[stage * MAX_SEG + seg], parity)) {
                    if (++polls > WAIT_LIMIT) { gave_up = true; break; }
                }
                ++seg;
                next_wait_tile += tl.tiles_per_seg;
            }
            if (gave_up) break;
            const bool second_half = tile * 64 + 32 < K;   // the last tile of a K that is 32 mod 64 is half empty
            const uint4 w0 = *reinterpret_cast<const uint4*>(wp + w_off0);
            uint4 w1 = make_uint4(0, 0, 0, 0);
            if (second_half) w1 = *reinterpret_cast<const uint4*>(wp + w_off1);
#pragma unroll
            for (int mt = 0; mt < MT16; ++mt) {
                uint4 lo0, hi0, lo1 = make_uint4(0, 0, 0, 0), hi1 = make_uint4(0, 0, 0, 0);
                if (XMODE == 0) {
                    const __nv_bfloat16* r_lo = Xb + (size_t)min(mt * 16 + pg, M - 1) * ldx + tile * 64 + t * 8;
                    const __nv_bfloat16* r_hi = Xb + (size_t)min(mt * 16 + pg + 8, M - 1) * ldx + tile * 64 + t * 8;
                    lo0 = __ldg(reinterpret_cast<const uint4*>(r_lo));
                    hi0 = __ldg(reinterpret_cast<const uint4*>(r_hi));
                    if (second_half) {
                        lo1 = __ldg(reinterpret_cast<const uint4*>(r_lo + 32));
                        hi1 = __ldg(reinterpret_cast<const uint4*>(r_hi + 32));
                    }
                } else {
                    lo0 = *reinterpret_cast<const uint4*>(xp + swz(mt * 16 + pg, t));
                    hi0 = *reinterpret_cast<const uint4*>(xp + swz(mt * 16 + pg + 8, t));
                    if (second_half) {
                        lo1 = *reinterpret_cast<const uint4*>(xp + swz(mt * 16 + pg, 4 + t));
                        hi1 = *reinterpret_cast<const uint4*>(xp + swz(mt * 16 + pg + 8, 4 + t));
                    }
                }
                mma_bf16(acc[mt], lo0.x, hi0.x, lo0.y, hi0.y, w0.x, w0.y);
                mma_bf16(acc[mt], lo0.z, hi0.z, lo0.w, hi0.w, w0.z, w0.w);
                mma_bf16(acc[mt], lo1.x, hi1.x, lo1.y, hi1.y, w1.x, w1.y);
                mma_bf16(acc[mt], lo1.z, hi1.z, lo1.w, hi1.w, w1.z, w1.w);
            }
        }

        // partial sums of the k-parts go through shared memory (two buffers in turn, so that one barrier a
        // group is enough) and are added in the order of the parts by the first warp of each 8-column group
        float* red_it = red + (size_t)(it & 1) * (SK_WARPS * MT16 * 4 * 32);
        float* mine = red_it + (size_t)warp * (MT16 * 4 * 32);
        if (wpg > 1) {
#pragma unroll
            for (int mt = 0; mt < MT16; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) mine[(mt * 4 + j) * 32 + lane] = acc[mt][j];
        }
        __syncthreads();                               // every warp is done with this stage's slab
        if (warp == 0 && it + S < n_my) {
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            request(it + S, false);
        }
        if (kpart != 0 || gave_up) continue;
        for (int p = 1; p < wpg; ++p) {
            const float* other = red_it + (size_t)(warp + p) * (MT16 * 4 * 32);
#pragma unroll
            for (int mt = 0; mt < MT16; ++mt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[mt][j] += other[(mt * 4 + j) * 32 + lane];
        }

        // epilogue: the thread holds rows mt*16 + pg, +8 and columns n0 + t, n0 + t + 4
#pragma unroll
        for (int mt = 0; mt < MT16; ++mt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int m = mt * 16 + pg + ((j & 2) ? 8 : 0);
                const int n = n0 + t + 4 * (j & 1);
                if (n >= N || m >= M) continue;
                float v = acc[mt][j] + pre_bias[j & 1];
                v = apply_act_out<OT>(v, act) + pre[mt][j];
                ElemIO<OT>::store(Y + (size_t)m * ldy + n, v);
                if (kv.Kc != nullptr && n >= kv.k_off) {
                    const bool is_v = n >= kv.v_off;
                    const int col = n - (is_v ? kv.v_off : kv.k_off);
                    const int blk = kv_blk[mt][(j & 2) ? 1 : 0];
                    if (col < kv.width && blk != -2) {
                        if (blk >= 0) {
                            const int h = col / kv.dh, cc = col - h * kv.dh;
                            const size_t dst = (((size_t)blk * kv.Hkv + h) * kv.BT + kv_off[mt][(j & 2) ? 1 : 0]) * kv.dh + cc;
                            __nv_bfloat16* base = reinterpret_cast<__nv_bfloat16*>(is_v ? kv.Vc : kv.Kc);
                            base[dst] = __float2bfloat16_rn(v);
                        } else {
                            atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
                        }
                    }
                }
            }
        }
    }
    if (gave_up && lane == 0) atomicOr(dev_err, VLRF_DEVERR_WAIT_TIMEOUT);
}

size_t smem_bytes(int MT16, int M, int xmode, int K, int CG, int S) {
    const Tiling tl = tiling(K);
    (void)M;
    return 1024 + (size_t)S * tl.n_tiles * 8 * CG * 128 + (xmode != 0 ? (size_t)tl.n_tiles * 16 * MT16 * 128 : 0) +
           (size_t)2 * SK_WARPS * MT16 * 4 * 32 * sizeof(float) + MAX_STAGES * MAX_SEG * 8;
}

constexpr size_t SMEM_LIMIT = 200 * 1024;

template <int MT16, int XMODE, typename OT>
int launch(const void* X, const void* W, const float* bias, const float* residual, void* Y, int M, int N, int K,
           int ldx, int ldy, int act, int CG, int S, int grid, const float* gamma, const float* beta, float eps,
           const KvScatter& kv, int* dev_err, cudaStream_t stream) {
    const size_t smem = smem_bytes(MT16, M, XMODE, K, CG, S);
    auto kern = gemm_skinny_kernel<MT16, XMODE, OT>;
    CUtensorMap tmap_w, tmap_x;
    int st = vlrf_make_tmap_bf16(W, N, K, K, 8 * CG, 64, &tmap_w);
    if (st != VLRF_OK) return st;
    if (XMODE == 1) {
        st = vlrf_make_tmap_bf16(X, M, K, ldx, 16 * MT16, 64, &tmap_x);
        if (st != VLRF_OK) return st;
    } else {
        tmap_x = tmap_w;   // unused
    }
    static size_t allowed = 48 * 1024;   // per instantiation: the attribute is raised once, not per launch
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_skinny: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        allowed = smem;
    }
    cudaError_t e = launch_chained(kern, dim3(grid), dim3(SK_THREADS), smem, stream, tmap_w, tmap_x, X, bias, residual,
                                   (OT*)Y, M, N, K, ldx, ldy, act, CG, S, gamma, beta, eps, kv, dev_err);
    if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "gemm_skinny: %s", cudaGetErrorString(e));
    return vlrf_check_launch("gemm_skinny");
}

template <int XMODE, typename OT>
int dispatch_mt(int mt16, const void* X, const void* W, const float* bias, const float* residual, void* Y, int M,
                int N, int K, int ldx, int ldy, int act, int CG, int S, int grid, const float* gamma, const float* beta,
                float eps, const KvScatter& kv, int* dev_err, cudaStream_t stream) {
    switch (mt16) {
        case 1: return launch<1, XMODE, OT>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, CG, S, grid, gamma, beta, eps, kv, dev_err, stream);
        case 2: return launch<2, XMODE, OT>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, CG, S, grid, gamma, beta, eps, kv, dev_err, stream);
        default: return launch<4, XMODE, OT>(X, W, bias, residual, Y, M, N, K, ldx, ldy, act, CG, S, grid, gamma, beta, eps, kv, dev_err, stream);
    }
}

int tiles16(int M) { return M <= 16 ? 1 : (M <= 32 ? 2 : 4); }
}  // namespace

// Whether the LayerNorm-fused form holds M normalised rows of width K in shared memory.
extern "C" int vlrf_gemm_skinny_ln_fits(int M, int K) {
    if (M < 1 || M > 64 || K % 32 != 0) return 0;
    return smem_bytes(tiles16(M), M, 2, K, 1, 1) <= SMEM_LIMIT ? 1 : 0;
}

extern "C" int vlrf_gemm_skinny(const void* X, int x_is_f32_ln, const void* W, const float* bias,
                                const float* residual, void* Y, int out_dtype, int M, int N, int K, int ldx,
                                int ldy, int act, const float* gamma, const float* beta, float eps,
                                // optional scatter of K/V columns into the cache (Kc == nullptr: none)
                                void* Kc, void* Vc, const int* block_table, int max_blocks, const int* tok_slot,
                                const int* tok_pos, int k_off, int v_off, int Hkv, int dh, int BT,
                                int sm_count, int* dev_err, cudaStream_t stream) {
    VLRF_REQUIRE(M >= 1 && M <= 64, "gemm_skinny: takes 1…64 rows, not %d", M);
    VLRF_REQUIRE(N > 0 && K > 0 && K % 32 == 0, "gemm_skinny: K=%d must be a positive multiple of 32", K);
    VLRF_REQUIRE(ldx >= K && ldy >= N, "gemm_skinny: leading sizes too small");
    VLRF_REQUIRE(act >= 0 && act <= 2, "gemm_skinny: unknown activation %d", act);
    VLRF_REQUIRE(x_is_f32_ln || ldx % 8 == 0, "gemm_skinny: bf16 rows must start on 16-byte boundaries (ldx=%d)", ldx);
    
    VLRF_REQUIRE(dev_err != nullptr, "gemm_skinny: needs the device error word");
    VLRF_REQUIRE(!x_is_f32_ln || (gamma && beta), "gemm_skinny: the fused LayerNorm needs weight and bias");
    VLRF_REQUIRE(!x_is_f32_ln || vlrf_gemm_skinny_ln_fits(M, K), "gemm_skinny: %d rows of width %d do not fit the fused LayerNorm", M, K);
    VLRF_REQUIRE(smem_bytes(1, 1, 0, K, 1, 1) <= SMEM_LIMIT, "gemm_skinny: K=%d is too wide for shared memory", K);
    KvScatter kv{};
    if (Kc != nullptr) {
        VLRF_REQUIRE(Vc && block_table && tok_slot && tok_pos && Hkv > 0 && dh > 0 && BT > 0 && max_blocks > 0,
                     "gemm_skinny: incomplete cache scatter arguments");
        VLRF_REQUIRE(out_dtype == VLRF_BF16, "gemm_skinny: the cache scatter writes bfloat16");
        kv = KvScatter{Kc, Vc, block_table, tok_slot, tok_pos, max_blocks, k_off, v_off, Hkv * dh, dh, Hkv, BT};
    }
    const int mt16 = tiles16(M);
    // X in shared memory when it fits beside a slab; else read per fragment through L1/L2
    int xmode = x_is_f32_ln ? 2 : ((size_t)tiling(K).n_tiles * 16 * mt16 * 128 <= 100 * 1024 ? 1 : 0);
    if (smem_bytes(mt16, M, xmode, K, 1, 1) > SMEM_LIMIT) {
        VLRF_REQUIRE(xmode != 2, "gemm_skinny: fused LayerNorm does not fit");
        xmode = 0;
    }
    // 8·CG rows of W per group.  These products are short: a CTA's time is a fixed latency (request, HBM
    // round trip, reduction, epilogue) plus its slab's bytes over the bandwidth it gets, times the rounds it
    // has to make.  The estimate below picks the group size with the least of that.
    int CG = 1;
    double best = 1e30;
    for (int cg = SK_WARPS; cg >= 1; cg /= 2) {
        const double slab = (double)8 * cg * tiling(K).n_tiles * 128;
        if (cg > 1 && slab > 64 * 1024) continue;
        if (smem_bytes(mt16, M, xmode, K, cg, 1) > SMEM_LIMIT) continue;
        const int groups = (N + 8 * cg - 1) / (8 * cg);
        const int ctas = groups < sm_count ? groups : sm_count;
        const int rounds = (groups + ctas - 1) / ctas;
        const double gbs = 6500.0 / ctas < 100.0 ? 6500.0 / ctas : 100.0;      // GB/s a CTA gets
        const double cost = rounds * (1.2 + slab / (gbs * 1e3));               // microseconds
        if (cost < best - 1e-9) { best = cost; CG = cg; }
    }
    const int groups = (N + 8 * CG - 1) / (8 * CG);
    const int grid = groups < sm_count ? groups : sm_count;
    const int rounds = (groups + grid - 1) / grid;
    int S = rounds < MAX_STAGES ? rounds : MAX_STAGES;
    while (S > 1 && smem_bytes(mt16, M, xmode, K, CG, S) > SMEM_LIMIT) --S;
    const int grid_x = grid;
#define GO(XM, OT) return dispatch_mt<XM, OT>(mt16, X, W, bias, residual, Y, M, N, K, ldx, ldy, act, CG, S, grid_x, gamma, beta, eps, kv, dev_err, stream)
    if (out_dtype == VLRF_BF16) {
        if (xmode == 2) GO(2, __nv_bfloat16);
        if (xmode == 1) GO(1, __nv_bfloat16);
        GO(0, __nv_bfloat16);
    }
    if (out_dtype == VLRF_F32) {
        if (xmode == 2) GO(2, float);
        if (xmode == 1) GO(1, float);
        GO(0, float);
    }
#undef GO
    return vlrf_fail(VLRF_ERR_INVALID_ARG, "gemm_skinny: unknown output dtype %d", out_dtype);
}
