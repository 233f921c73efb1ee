// Cache append and the general attention kernel over the paged cache.
//
// The cache of one layer is K and V of shape [block][kv_head][BT][head_dim]; a sequence's slot maps its
// positions to blocks through block_table[slot][pos / BT].  `kv_append` scatters the K and V columns of
// the fused projection into place (reference: include/model/kv_cache.hpp:215-251, before attention at
// include/model/attention.hpp:127-129).  `attn_generic` serves any mix of tokens: each (token, head) is
// one warp that walks the keys 0…pos of its slot in chunks of 32 with an online softmax in float32
// (reference: include/model/attention.hpp:207-309; scale :373-374; key visible iff k ≤ position
// :253-260).  It is the attention of the 32-bit path for prefill and decode, takes every head size that
// is a multiple of 16 up to 256 and any number of heads and groups, and is the fallback of the bfloat16
// path.  A window w > 0 hides keys at or before position − w.
#include "common.cuh"

namespace {

template <typename ET>
__global__ void kv_append_kernel(const ET* __restrict__ qkv, int ld, int k_off, int v_off,
                                 ET* __restrict__ Kc, ET* __restrict__ Vc,
                                 const int* __restrict__ block_table, int max_blocks,
                                 const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                                 int Hkv, int dh, int BT, int* __restrict__ dev_err) {
    const int t = blockIdx.x;
    const int slot = tok_slot[t];
    if (slot < 0) return;  // padding row
    const int pos = tok_pos[t];
    const int bi = pos / BT;
    const int blk = (pos >= 0 && bi < max_blocks) ? block_table[(size_t)slot * max_blocks + bi] : -1;
    if (blk < 0) {
        if (threadIdx.x == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
        return;
    }
    const int width = Hkv * dh;
    const ET* src = qkv + (size_t)t * ld;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int h = i / dh, c = i - h * dh;
        const size_t dst = (((size_t)blk * Hkv + h) * BT + (pos % BT)) * dh + c;
        Kc[dst] = src[k_off + i];
        Vc[dst] = src[v_off + i];
    }
}

template <typename ET> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float* out) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
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

constexpr int ATT_WARPS = 4;
constexpr int MAX_DH = 256;

template <typename ET>
__global__ void __launch_bounds__(ATT_WARPS * 32)
attn_generic_kernel(const ET* __restrict__ qkv, int ld, int q_off, const ET* __restrict__ Kc,
                    const ET* __restrict__ Vc, const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ tok_slot, const int* __restrict__ tok_pos,
                    ET* __restrict__ out, int ld_out, int H, int Hkv, int dh, int BT, float scale,
                    int window, int* __restrict__ dev_err) {
    extern __shared__ float q_sm[];  // [ATT_WARPS][dh]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int h = blockIdx.y * ATT_WARPS + warp;
    const int slot = tok_slot[t];
    if (h >= H || slot < 0) return;  // whole warp leaves together; no block-wide barrier below
    const int pos = tok_pos[t];
    const int hk = h / (H / Hkv);
    float* q = q_sm + warp * dh;
    const ET* qsrc = qkv + (size_t)t * ld + q_off + (size_t)h * dh;
    for (int i = lane; i < dh; i += 32) q[i] = ElemIO<ET>::load(qsrc + i) * scale;
    __syncwarp();

    float acc[MAX_DH / 32];
#pragma unroll
    for (int i = 0; i < MAX_DH / 32; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int first = (window > 0) ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)slot * max_blocks;
    bool lost = false;

    for (int k0 = (first / 32) * 32; k0 <= pos; k0 += 32) {
        const int blk = table[k0 / BT];
        if (blk < 0) { lost = true; break; }
        const size_t base = (((size_t)blk * Hkv + hk) * BT + (k0 % BT)) * dh;
        const int key = k0 + lane;
        const bool valid = key >= first && key <= pos;
        float s = -INFINITY;
        if (valid) {
            const ET* krow = Kc + base + (size_t)lane * dh;
            float dot = 0.f;
            for (int c = 0; c < dh; c += Vec16<ET>::N) {
                float kv[Vec16<ET>::N];
                Vec16<ET>::load(krow + c, kv);
#pragma unroll
                for (int j = 0; j < Vec16<ET>::N; ++j) dot = fmaf(q[c + j], kv[j], dot);
            }
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));      // at least one key of the chunk is valid
        const float p = valid ? expf(s - m_new) : 0.f;
        const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_DH / 32; ++i) acc[i] *= corr;
        const int n_here = min(32, pos - k0 + 1);
        const ET* vbase = Vc + base;
        for (int j = 0; j < n_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            if (pj == 0.f) continue;  // uniform across the warp
            const ET* vrow = vbase + (size_t)j * dh;
#pragma unroll
            for (int i = 0; i < MAX_DH / 32; ++i) {
                const int c = i * 32 + lane;
                if (c < dh) acc[i] = fmaf(pj, ElemIO<ET>::load(vrow + c), acc[i]);
            }
        }
        m = m_new;
    }
    if (lost && lane == 0) atomicOr(dev_err, VLRF_DEVERR_NO_BLOCK);
    const float inv = (l > 0.f) ? 1.f / l : 0.f;
    ET* dst = out + (size_t)t * ld_out + (size_t)h * dh;
#pragma unroll
    for (int i = 0; i < MAX_DH / 32; ++i) {
        const int c = i * 32 + lane;
        if (c < dh) ElemIO<ET>::store(dst + c, acc[i] * inv);
    }
}
}  // namespace

extern "C" int vlrf_kv_append(const void* qkv, int dtype, int ld, int k_off, int v_off, void* Kc, void* Vc,
                              const int* block_table, int max_blocks, const int* tok_slot,
                              const int* tok_pos, int T, int Hkv, int dh, int BT, int* dev_err,
                              cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && Hkv > 0 && dh > 0 && BT > 0 && max_blocks > 0, "kv_append: bad sizes");
    VLRF_REQUIRE(dev_err != nullptr, "kv_append: needs the device error word");
    if (T == 0) return VLRF_OK;
    const int threads = (Hkv * dh >= 256) ? 256 : 128;
    if (dtype == VLRF_F32)
        kv_append_kernel<float><<<T, threads, 0, stream>>>((const float*)qkv, ld, k_off, v_off, (float*)Kc,
                                                          (float*)Vc, block_table, max_blocks, tok_slot,
                                                          tok_pos, Hkv, dh, BT, dev_err);
    else if (dtype == VLRF_BF16)
        kv_append_kernel<__nv_bfloat16><<<T, threads, 0, stream>>>(
            (const __nv_bfloat16*)qkv, ld, k_off, v_off, (__nv_bfloat16*)Kc, (__nv_bfloat16*)Vc,
            block_table, max_blocks, tok_slot, tok_pos, Hkv, dh, BT, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "kv_append: unknown dtype %d", dtype);
    return vlrf_check_launch("kv_append");
}

extern "C" int vlrf_attn_generic(const void* qkv, int dtype, int ld, int q_off, const void* Kc,
                                 const void* Vc, const int* block_table, int max_blocks,
                                 const int* tok_slot, const int* tok_pos, void* out, int ld_out, int T,
                                 int H, int Hkv, int dh, int BT, float scale, int window, int* dev_err,
                                 cudaStream_t stream) {
    VLRF_REQUIRE(T >= 0 && H > 0 && Hkv > 0 && max_blocks > 0, "attention: bad sizes");
    VLRF_REQUIRE(H % Hkv == 0, "attention: %d heads cannot share %d key/value heads", H, Hkv);
    VLRF_REQUIRE(dh > 0 && dh % 16 == 0 && dh <= MAX_DH,
                 "attention: head size %d is not a multiple of 16 up to %d", dh, MAX_DH);
    VLRF_REQUIRE(BT % 32 == 0, "attention: cache blocks of %d tokens are not a multiple of 32", BT);
    VLRF_REQUIRE(window >= 0, "attention: negative window");
    VLRF_REQUIRE(dev_err != nullptr, "attention: needs the device error word");
    if (T == 0) return VLRF_OK;
    dim3 grid(T, (H + ATT_WARPS - 1) / ATT_WARPS);
    const size_t smem = (size_t)ATT_WARPS * dh * sizeof(float);
    if (dtype == VLRF_F32)
        attn_generic_kernel<float><<<grid, ATT_WARPS * 32, smem, stream>>>(
            (const float*)qkv, ld, q_off, (const float*)Kc, (const float*)Vc, block_table, max_blocks,
            tok_slot, tok_pos, (float*)out, ld_out, H, Hkv, dh, BT, scale, window, dev_err);
    else if (dtype == VLRF_BF16)
        attn_generic_kernel<__nv_bfloat16><<<grid, ATT_WARPS * 32, smem, stream>>>(
            (const __nv_bfloat16*)qkv, ld, q_off, (const __nv_bfloat16*)Kc, (const __nv_bfloat16*)Vc,
            block_table, max_blocks, tok_slot, tok_pos, (__nv_bfloat16*)out, ld_out, H, Hkv, dh, BT, scale,
            window, dev_err);
    else
        return vlrf_fail(VLRF_ERR_INVALID_ARG, "attention: unknown dtype %d", dtype);
    return vlrf_check_launch("attn_generic");
}
