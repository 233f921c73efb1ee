// Sampling on the device: one block per row of float32 logits.
//
// Order of operations as in the reference's sampler (include/model/transformer.hpp:124-182):
// temperature ≤ 0 (or a greedy row) → first maximal index (:43-47); else logits/temperature → softmax →
// keep the top_k most probable → walk by descending probability and cut the first token whose running
// mass exceeds top_p together with all after it, the most probable always staying (:159-165) →
// renormalise → draw the first index whose cumulative probability reaches the uniform number u (:175-181).
// Penalties on generated tokens and the n-gram block (:54-120) are a kernel of their own that edits the
// logits first.
//
// Nothing is sorted.  The cut is found by a radix select over the float bits of the unnormalised
// probabilities e_i = exp((l_i − max)/T), 8 bits a pass, with per-bin counts and masses; masses are
// summed as 32.32 fixed-point integers so that every sum is exact and independent of the order in which
// threads add — the same seed gives the same token on every run.  Equal probabilities at the cut are kept
// in index order (the reference leaves their order to std::sort / std::partial_sort).
//
// The uniform number of a row is a counter-based hash of (rng_key[row], rng_ctr[row]); the counter
// advances by one per draw, so a request's stream depends on nothing but its key and how many tokens it
// drew.
#include "common.cuh"

namespace {
constexpr int ST = 1024;  // threads per row

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
    x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
    x ^= x >> 27; x *= 0x94D049BB133111EBull;
    x ^= x >> 31;
    return x;
}
// u in [0,1) with 24 bits
__device__ __forceinline__ float uniform01(unsigned long long key, unsigned int ctr) {
    const unsigned long long x = mix64(key + 0x9E3779B97F4A7C15ull * (unsigned long long)(ctr + 1u));
    return (float)(x >> 40) * (1.0f / 16777216.0f);
}

struct ArgMax { float v; int i; };
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}
__device__ ArgMax block_argmax(ArgMax a, ArgMax* sm /*32*/) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) sm[warp] = a;
    __syncthreads();
    ArgMax r = sm[0];
    for (int w = 1; w < ST / 32; ++w) r = better(r, sm[w]);
    return r;
}

// exclusive block scan; returns this thread's prefix and writes the total
template <typename T>
__device__ T block_excl_scan(T v, T* sm /*32*/, T* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        T n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) sm[warp] = inc;
    __syncthreads();
    T base = 0, tot = 0;
    for (int w = 0; w < ST / 32; ++w) {
        if (w < warp) base += sm[w];
        tot += sm[w];
    }
    *total = tot;
    return base + inc - v;
}

__device__ __forceinline__ float unnorm_prob(float logit, float mx, float inv_t) {
    return expf((logit - mx) * inv_t);
}
__device__ __forceinline__ unsigned long long to_fixed(float e) {  // e in [0,1] → 32.32 (the scaling is exact)
    return __float2ull_rz(e * 4294967296.0f);
}
__global__ void __launch_bounds__(ST)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const unsigned long long* __restrict__ rng_key, unsigned int* __restrict__ rng_ctr,
              int* __restrict__ out_token, int* __restrict__ next_token, int* __restrict__ next_pos,
              const int* __restrict__ row_slot) {
    __shared__ ArgMax sm_am[32];
    __shared__ unsigned long long sm_u64[32];
    __shared__ int sm_i32[32];
    __shared__ unsigned int h_cnt[256];
    __shared__ unsigned long long h_mass[256];
    __shared__ unsigned int s_prefix;
    __shared__ unsigned int s_cnt_above;
    __shared__ unsigned long long s_mass_above;
    __shared__ int s_hit;
    __shared__ int s_choice;

    const int row = blockIdx.x, tid = threadIdx.x;
    pdl_wait();
    pdl_launch_dependents();
    const float* lg = logits + (size_t)row * ld;

    ArgMax am{-INFINITY, 0x7fffffff};
    for (int i = tid; i < V; i += ST) {
        const float v = lg[i];
        if (v > am.v) { am.v = v; am.i = i; }
    }
    am = block_argmax(am, sm_am);
    if (am.i == 0x7fffffff) am.i = 0;  // a row of NaNs or −inf: defined answer
    const float temp = temperature ? temperature[row] : 0.f;
    if (!(temp > 0.f)) {
        if (tid == 0) {
            out_token[row] = am.i;
            // feed the next step on the device: the token becomes the row's input, its position moves on
            if (next_token) next_token[row] = am.i;
            if (next_pos && (!row_slot || row_slot[row] >= 0)) next_pos[row] += 1;
        }
        return;
    }
    const float mx = am.v, inv_t = 1.f / temp;

    // total unnormalised mass
    unsigned long long part = 0;
    for (int i = tid; i < V; i += ST) part += to_fixed(unnorm_prob(lg[i], mx, inv_t));
    unsigned long long total = 0;
    block_excl_scan<unsigned long long>(part, sm_u64, &total);

    const int k_in = top_k ? top_k[row] : 0;
    const unsigned int k_eff = (k_in > 0 && k_in < V) ? (unsigned int)k_in : (unsigned int)V;
    const float tp = top_p ? top_p[row] : 1.f;
    const bool use_p = tp < 1.f;
    const unsigned long long thresh =
        use_p ? (unsigned long long)((double)fmaxf(tp, 0.f) * (double)total) : ~0ull;

    // ---- radix select of the cut value -------------------------------------------------------
    bool keep_all = (k_eff >= (unsigned int)V) && !use_p;
    unsigned int cut_bits = 0, ties_kept = 0;
    if (!keep_all) {
        if (tid == 0) { s_prefix = 0; s_cnt_above = 0; s_mass_above = 0; }
        unsigned int mask = 0;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = tid; b < 256; b += ST) { h_cnt[b] = 0; h_mass[b] = 0; }
            __syncthreads();
            const unsigned int prefix = s_prefix;
            for (int i = tid; i < V; i += ST) {
                const float e = unnorm_prob(lg[i], mx, inv_t);
                const unsigned int bits = __float_as_uint(e);
                if ((bits & mask) == prefix) {
                    const unsigned int bin = (bits >> shift) & 255u;
                    atomicAdd(&h_cnt[bin], 1u);
                    atomicAdd(&h_mass[bin], to_fixed(e));
                }
            }
            __syncthreads();
            if (tid == 0) {
                unsigned int c = s_cnt_above;
                unsigned long long ms = s_mass_above;
                int hit = 0;
                for (int b = 255; b >= 0; --b) {
                    if (h_cnt[b] == 0) continue;
                    const unsigned int c2 = c + h_cnt[b];
                    const unsigned long long ms2 = ms + h_mass[b];
                    if (c2 >= k_eff || ms2 > thresh) {
                        s_prefix = prefix | ((unsigned int)b << shift);
                        hit = 1;
                        break;
                    }
                    c = c2; ms = ms2;
                }
                s_cnt_above = c; s_mass_above = ms; s_hit = hit;
            }
            __syncthreads();
            if (!s_hit) { keep_all = true; break; }  // uniform: read from shared memory
            mask |= 255u << shift;
        }
        if (!keep_all) {
            cut_bits = s_prefix;
            const unsigned int above = s_cnt_above;
            const unsigned long long e_cut = to_fixed(__uint_as_float(cut_bits));
            unsigned long long by_p = ~0ull;
            if (use_p && e_cut > 0) by_p = (thresh >= s_mass_above) ? (thresh - s_mass_above) / e_cut : 0ull;
            if (above == 0 && by_p == 0) by_p = 1;  // the most probable token always stays
            unsigned long long by_k = (unsigned long long)(k_eff - above);  // above < k_eff by construction
            ties_kept = (unsigned int)min(by_p, by_k);
        }
    }

    // ---- draw in index order over what is kept ---------------------------------------------------
    const int chunk = (V + ST - 1) / ST;
    const int i0 = min(V, tid * chunk), i1 = min(V, i0 + chunk);
    int my_ties = 0;
    if (!keep_all)
        for (int i = i0; i < i1; ++i)
            my_ties += (__float_as_uint(unnorm_prob(lg[i], mx, inv_t)) == cut_bits);
    int ties_total = 0;
    const int tie_base = block_excl_scan<int>(my_ties, sm_i32, &ties_total);

    unsigned long long my_mass = 0;
    {
        int seen = tie_base;
        for (int i = i0; i < i1; ++i) {
            const float e = unnorm_prob(lg[i], mx, inv_t);
            bool keep = true;
            if (!keep_all) {
                const unsigned int bits = __float_as_uint(e);
                if (bits == cut_bits) { keep = (unsigned int)seen < ties_kept; ++seen; }
                else keep = bits > cut_bits;
            }
            if (keep) my_mass += to_fixed(e);
        }
    }
    unsigned long long kept_total = 0;
    const unsigned long long mass_base = block_excl_scan<unsigned long long>(my_mass, sm_u64, &kept_total);
    if (tid == 0) s_choice = -1;
    __syncthreads();
    if (kept_total == 0) {  // nothing left to draw from (:169-172): the maximal logit
        if (tid == 0) out_token[row] = am.i;
    } else {
        const unsigned int ctr = rng_ctr[row];
        const float u = uniform01(rng_key[row], ctr);
        unsigned long long tgt = (unsigned long long)((double)u * (double)kept_total) + 1ull;
        if (tgt > kept_total) tgt = kept_total;
        if (my_mass > 0 && mass_base < tgt && tgt <= mass_base + my_mass) {
            unsigned long long cum = mass_base;
            int seen = tie_base;
            for (int i = i0; i < i1; ++i) {
                const float e = unnorm_prob(lg[i], mx, inv_t);
                bool keep = true;
                if (!keep_all) {
                    const unsigned int bits = __float_as_uint(e);
                    if (bits == cut_bits) { keep = (unsigned int)seen < ties_kept; ++seen; }
                    else keep = bits > cut_bits;
                }
                if (keep) {
                    cum += to_fixed(e);
                    if (cum >= tgt) { s_choice = i; break; }
                }
            }
        }
        __syncthreads();
        if (tid == 0) out_token[row] = (s_choice >= 0) ? s_choice : am.i;
    }
    __syncthreads();
    if (tid == 0) {
        rng_ctr[row] = rng_ctr[row] + 1u;
        if (next_token) next_token[row] = out_token[row];
        if (next_pos && (!row_slot || row_slot[row] >= 0)) next_pos[row] += 1;
    }
}

// ---------------------------------------------------------------------------------------------------------
// The same sampler with a row spread over a cluster of SC CTAs: CTA r owns the indices [r·S, (r+1)·S) and keeps
// their e_i in shared memory, so that exp runs once per logit and the passes of the radix select read shared
// memory.  What the CTAs exchange — maxima, masses, the 256-bin histograms of a pass, tie counts — they read
// from one another's shared memory after a cluster barrier; every CTA then makes the same decision with the
// same integer arithmetic.  Same order of operations, same fixed-point masses and same tie rule as above: the
// two kernels choose the same token.
constexpr int SC = 8;      // CTAs of a row
constexpr int STC = 256;   // threads of a CTA

__device__ __forceinline__ unsigned int ld_cluster_u32(const void* own, unsigned int rank) {
    unsigned int remote, v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((unsigned int)__cvta_generic_to_shared(own)), "r"(rank));
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long ld_cluster_u64(const void* own, unsigned int rank) {
    unsigned int remote;
    unsigned long long v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"((unsigned int)__cvta_generic_to_shared(own)), "r"(rank));
    asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(remote) : "memory");
    return v;
}
// inclusive scan over the STC threads of a CTA (all must call); sm: STC/32 values
template <typename T>
__device__ T cta_incl_scan(T v, T* sm, T* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    T inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        T n = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += n;
    }
    __syncthreads();
    if (lane == 31) sm[warp] = inc;
    __syncthreads();
    T base = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < STC / 32; ++w) {
        if (w < warp) base += sm[w];
        tot += sm[w];
    }
    *total = tot;
    return base + inc;
}

__global__ void __launch_bounds__(STC)
sample_cluster_kernel(const float* __restrict__ logits, int ld, int V, int S, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p,
                      const unsigned long long* __restrict__ rng_key, unsigned int* __restrict__ rng_ctr,
                      int* __restrict__ out_token, int* __restrict__ next_token, int* __restrict__ next_pos,
                      const int* __restrict__ row_slot) {
    extern __shared__ unsigned int e_bits[];                  // [S] float bits of e_i of this CTA's indices
    // A histogram of its own for every warp, [warp][256 bins][count, mass low word, mass high word]: shared
    // memory adds 32-bit integers natively (a 64-bit add would be a compare-and-swap loop), and the few bins of
    // the first pass would make all warps queue on the same words.
    unsigned int* wh = e_bits + S;
    __shared__ ArgMax sm_am[STC / 32];
    __shared__ unsigned long long sm_u64[STC / 32];
    __shared__ int sm_i32[STC / 32];
    __shared__ unsigned int sm_u32[STC / 32];
    __shared__ unsigned int h_cnt[2][256];                    // two in turn: a neighbour may still read the last pass's
    __shared__ unsigned long long h_mass[2][256];
    __shared__ float x_max; __shared__ int x_arg;             // what the other CTAs of the cluster read
    __shared__ unsigned long long x_total, x_kept;
    __shared__ int x_ties;
    __shared__ unsigned int d_prefix, d_cnt_above; __shared__ unsigned long long d_mass_above; __shared__ int d_hit;

    const int tid = threadIdx.x;
    const unsigned int rank = blockIdx.x % SC;
    const int row = blockIdx.x / SC;
    pdl_wait();
    pdl_launch_dependents();
    const float* lg = logits + (size_t)row * ld;
    const int lo = min(V, (int)rank * S), hi = min(V, lo + S);      // this CTA's indices
    const int n_mine = hi - lo;

    // ---- the maximum and its first index ----
    ArgMax am{-INFINITY, 0x7fffffff};
    for (int i = lo + tid; i < hi; i += STC) {
        const float v = lg[i];
        if (v > am.v) { am.v = v; am.i = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, am.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, am.i, o);
        am = better(am, b);
    }
    if ((tid & 31) == 0) sm_am[tid >> 5] = am;
    __syncthreads();
    if (tid == 0) {
        ArgMax r = sm_am[0];
        for (int w = 1; w < STC / 32; ++w) r = better(r, sm_am[w]);
        x_max = r.v; x_arg = r.i;
    }
    cluster_sync_all();
    am = ArgMax{-INFINITY, 0x7fffffff};
    {
        unsigned int vr[SC], ir[SC];
#pragma unroll
        for (unsigned int r = 0; r < SC; ++r) { vr[r] = ld_cluster_u32(&x_max, r); ir[r] = ld_cluster_u32(&x_arg, r); }
#pragma unroll
        for (unsigned int r = 0; r < SC; ++r) am = better(am, ArgMax{__uint_as_float(vr[r]), (int)ir[r]});
    }
    if (am.i == 0x7fffffff) am.i = 0;                          // a row of NaNs or −inf: defined answer
    const float temp = temperature ? temperature[row] : 0.f;
    const bool greedy = !(temp > 0.f);                        // uniform over the cluster
    const float mx = am.v, inv_t = greedy ? 0.f : 1.f / temp;

    unsigned long long total = 0, kept_total = 0, mass_base = 0, my_mass = 0, mass_in_cta = 0;
    unsigned int cut_bits = 0, ties_kept = 0;
    bool keep_all = true;
    int tie_base = 0;
    const int chunk = (S + STC - 1) / STC;                    // a thread's contiguous piece of the slice, for the draw
    const int j0 = min(n_mine, tid * chunk), j1 = min(n_mine, j0 + chunk);
    if (!greedy) {
        // ---- e_i once, kept in shared memory; the total mass ----
        unsigned long long part = 0;
        for (int j = tid; j < n_mine; j += STC) {
            const float e = unnorm_prob(lg[lo + j], mx, inv_t);
            e_bits[j] = __float_as_uint(e);
            part += to_fixed(e);
        }
        unsigned long long mine_total = 0;
        cta_incl_scan<unsigned long long>(part, sm_u64, &mine_total);
        if (tid == 0) x_total = mine_total;
        cluster_sync_all();
        {
            unsigned long long tr[SC];
#pragma unroll
            for (unsigned int r = 0; r < SC; ++r) tr[r] = ld_cluster_u64(&x_total, r);
#pragma unroll
            for (unsigned int r = 0; r < SC; ++r) total += tr[r];
        }

        const int k_in = top_k ? top_k[row] : 0;
        const unsigned int k_eff = (k_in > 0 && k_in < V) ? (unsigned int)k_in : (unsigned int)V;
        const float tp = top_p ? top_p[row] : 1.f;
        const bool use_p = tp < 1.f;
        const unsigned long long thresh = use_p ? (unsigned long long)((double)fmaxf(tp, 0.f) * (double)total) : ~0ull;
        keep_all = (k_eff >= (unsigned int)V) && !use_p;

        // ---- radix select of the cut value: every CTA adds up all histograms and decides alike ----
        if (!keep_all) {
            unsigned int prefix = 0, mask = 0, cnt_above = 0;
            unsigned long long mass_above = 0;
            int pass = 0;
            for (int shift = 24; shift >= 0; shift -= 8, ++pass) {
                unsigned int* hc = h_cnt[pass & 1];
                unsigned long long* hm = h_mass[pass & 1];
                for (int i = tid; i < (STC / 32) * 256 * 3; i += STC) wh[i] = 0;
                __syncthreads();
                unsigned int* mine = wh + (tid >> 5) * (256 * 3);
                for (int j = tid; j < n_mine; j += STC) {
                    const unsigned int bits = e_bits[j];
                    if ((bits & mask) == prefix) {
                        unsigned int* slot = mine + ((bits >> shift) & 255u) * 3;
                        const unsigned long long m = to_fixed(__uint_as_float(bits));
                        const unsigned int lo32 = (unsigned int)m, hi32 = (unsigned int)(m >> 32);
                        atomicAdd(&slot[0], 1u);
                        const unsigned int old = atomicAdd(&slot[1], lo32);          // the low word first; a wrap-around carries
                        const unsigned int carry = (old + lo32 < old) ? 1u : 0u;
                        if (hi32 + carry) atomicAdd(&slot[2], hi32 + carry);
                    }
                }
                __syncthreads();
                {                                              // the warps' histograms into the CTA's: bin tid (STC == 256)
                    unsigned int c = 0;
                    unsigned long long ms = 0;
#pragma unroll
                    for (int w = 0; w < STC / 32; ++w) {
                        const unsigned int* slot = wh + w * (256 * 3) + tid * 3;
                        c += slot[0];
                        ms += ((unsigned long long)slot[2] << 32) + slot[1];
                    }
                    hc[tid] = c; hm[tid] = ms;
                }
                cluster_sync_all();
                // bin b = 255 − tid, so that an inclusive scan runs from the largest values down
                const int b = 255 - tid;
                unsigned int c = 0, cr[SC];
                unsigned long long ms = 0, mr[SC];
#pragma unroll
                for (unsigned int r = 0; r < SC; ++r) { cr[r] = ld_cluster_u32(&hc[b], r); mr[r] = ld_cluster_u64(&hm[b], r); }   // all in flight
#pragma unroll
                for (unsigned int r = 0; r < SC; ++r) { c += cr[r]; ms += mr[r]; }
                unsigned int c_tot; unsigned long long m_tot;
                const unsigned int c_inc = cnt_above + cta_incl_scan<unsigned int>(c, sm_u32, &c_tot);
                const unsigned long long m_inc = mass_above + cta_incl_scan<unsigned long long>(ms, sm_u64, &m_tot);
                const bool now = c_inc >= k_eff || m_inc > thresh;
                const bool before = (c_inc - c) >= k_eff || (m_inc - ms) > thresh;
                if (tid == 0) d_hit = 0;
                __syncthreads();
                if (c > 0 && now && !before) {                 // the one bin where the cut falls
                    d_prefix = prefix | ((unsigned int)b << shift);
                    d_cnt_above = c_inc - c; d_mass_above = m_inc - ms; d_hit = 1;
                }
                __syncthreads();
                if (!d_hit) { keep_all = true; break; }        // the same in every CTA
                prefix = d_prefix; cnt_above = d_cnt_above; mass_above = d_mass_above;
                mask |= 255u << shift;
                __syncthreads();                               // d_* are read before the next pass writes them
            }
            if (!keep_all) {
                cut_bits = prefix;
                const unsigned long long e_cut = to_fixed(__uint_as_float(cut_bits));
                unsigned long long by_p = ~0ull;
                if (use_p && e_cut > 0) by_p = (thresh >= mass_above) ? (thresh - mass_above) / e_cut : 0ull;
                if (cnt_above == 0 && by_p == 0) by_p = 1;      // the most probable token always stays
                const unsigned long long by_k = (unsigned long long)(k_eff - cnt_above);
                ties_kept = (unsigned int)min(by_p, by_k);
            }
        }

        // ---- what is kept, in index order: ties first come first ----
        int my_ties = 0;
        if (!keep_all)
            for (int j = j0; j < j1; ++j) my_ties += (e_bits[j] == cut_bits);
        int ties_mine = 0;
        const int tie_in_cta = cta_incl_scan<int>(my_ties, sm_i32, &ties_mine) - my_ties;
        if (tid == 0) x_ties = ties_mine;
        cluster_sync_all();
        tie_base = tie_in_cta;
        {
            unsigned int tr[SC];
#pragma unroll
            for (unsigned int r = 0; r < SC; ++r) tr[r] = ld_cluster_u32(&x_ties, r);
#pragma unroll
            for (unsigned int r = 0; r < SC; ++r) tie_base += r < rank ? (int)tr[r] : 0;
        }
        {
            int seen = tie_base;
            for (int j = j0; j < j1; ++j) {
                const unsigned int bits = e_bits[j];
                bool keep = true;
                if (!keep_all) {
                    if (bits == cut_bits) { keep = (unsigned int)seen < ties_kept; ++seen; }
                    else keep = bits > cut_bits;
                }
                if (keep) my_mass += to_fixed(__uint_as_float(bits));
            }
        }
        unsigned long long kept_mine = 0;
        mass_in_cta = cta_incl_scan<unsigned long long>(my_mass, sm_u64, &kept_mine) - my_mass;
        if (tid == 0) x_kept = kept_mine;
    }
    // the fallback answer first (the maximal logit); the thread that finds the drawn token overwrites it
    if (rank == 0 && tid == 0) {
        out_token[row] = am.i;
        if (next_token) next_token[row] = am.i;
    }
    cluster_sync_all();
    if (!greedy) {
        mass_base = mass_in_cta;
        unsigned long long kr[SC];
#pragma unroll
        for (unsigned int r = 0; r < SC; ++r) kr[r] = ld_cluster_u64(&x_kept, r);
#pragma unroll
        for (unsigned int r = 0; r < SC; ++r) {
            if (r < rank) mass_base += kr[r];
            kept_total += kr[r];
        }
    }
    if (!greedy && kept_total > 0) {
        const float u = uniform01(rng_key[row], rng_ctr[row]);
        unsigned long long tgt = (unsigned long long)((double)u * (double)kept_total) + 1ull;
        if (tgt > kept_total) tgt = kept_total;
        if (my_mass > 0 && mass_base < tgt && tgt <= mass_base + my_mass) {
            unsigned long long cum = mass_base;
            int seen = tie_base;
            for (int j = j0; j < j1; ++j) {
                const unsigned int bits = e_bits[j];
                bool keep = true;
                if (!keep_all) {
                    if (bits == cut_bits) { keep = (unsigned int)seen < ties_kept; ++seen; }
                    else keep = bits > cut_bits;
                }
                if (keep) {
                    cum += to_fixed(__uint_as_float(bits));
                    if (cum >= tgt) {
                        out_token[row] = lo + j;
                        if (next_token) next_token[row] = lo + j;
                        break;
                    }
                }
            }
        }
    }
    cluster_sync_all();                                        // the token is written; nobody reads shared memory after this
    if (rank == 0 && tid == 0) {
        if (!greedy) rng_ctr[row] = rng_ctr[row] + 1u;
        if (next_pos && (!row_slot || row_slot[row] >= 0)) next_pos[row] += 1;
    }
}

// Penalties over the tokens a request generated so far, and the n-gram block
// (include/model/transformer.hpp:54-120).  One block per row; thread j looks at generated token j.
__global__ void penalties_kernel(float* __restrict__ logits, int ld, int V, const int* __restrict__ gen,
                                 int gen_ld, const int* __restrict__ gen_len,
                                 const float* __restrict__ rep, const float* __restrict__ freq,
                                 const float* __restrict__ pres, const int* __restrict__ ngram) {
    const int row = blockIdx.x;
    const int n = min(gen_len[row], gen_ld);       // a count beyond the row's width reads nothing beyond it
    if (n <= 0) return;
    const int* g = gen + (size_t)row * gen_ld;
    float* lg = logits + (size_t)row * ld;
    const float r = rep ? rep[row] : 1.f, f = freq ? freq[row] : 0.f, p = pres ? pres[row] : 0.f;
    if (r != 1.f || f != 0.f || p != 0.f) {
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            const int tok = g[j];
            if (tok < 0 || tok >= V) continue;
            bool first = true;
            for (int i = 0; i < j; ++i)
                if (g[i] == tok) { first = false; break; }
            if (!first) continue;  // the first occurrence speaks for all
            int count = 1;
            for (int i = j + 1; i < n; ++i) count += (g[i] == tok);
            float v = lg[tok];
            if (r != 1.f) v = (v > 0.f) ? v / r : v * r;
            if (f != 0.f) v -= f * (float)count;
            if (p != 0.f) v -= p;
            lg[tok] = v;
        }
    }
    __syncthreads();
    const int ng = ngram ? ngram[row] : 0;
    if (ng > 1 && n >= ng - 1) {
        const int* suffix = g + n - (ng - 1);
        for (int start = threadIdx.x; start + ng <= n; start += blockDim.x) {
            bool match = true;
            for (int k = 0; k < ng - 1; ++k)
                if (g[start + k] != suffix[k]) { match = false; break; }
            if (match) {
                const int forbidden = g[start + ng - 1];
                if (forbidden >= 0 && forbidden < V) lg[forbidden] = -INFINITY;
            }
        }
    }
}
}  // namespace

// next_token / next_pos / row_slot (all optional): after choosing, write the token into next_token[row] and
// add one to next_pos[row] (for rows whose slot is not −1), so that a decode step can be followed by the
// next without the host touching the tables.
extern "C" int vlrf_sample(const float* logits, int ld, int n_rows, int V, const float* temperature,
                           const int* top_k, const float* top_p, const unsigned long long* rng_key,
                           unsigned int* rng_ctr, int* out_token, int* next_token, int* next_pos,
                           const int* row_slot, cudaStream_t stream) {
    VLRF_REQUIRE(n_rows >= 0 && V > 0 && ld >= V, "sample: bad sizes rows=%d V=%d ld=%d", n_rows, V, ld);
    VLRF_REQUIRE(temperature == nullptr || (rng_key != nullptr && rng_ctr != nullptr),
                 "sample: temperature sampling needs the rows' random keys and counters");
    if (n_rows == 0) return VLRF_OK;
    // a cluster of CTAs a row, if a CTA's share of e_i fits its shared memory
    const int S = (V + SC - 1) / SC;
    const size_t smem = (size_t)S * sizeof(unsigned int) + (size_t)(STC / 32) * 256 * 3 * sizeof(unsigned int);
    if (smem <= 160 * 1024) {
        static size_t allowed = 48 * 1024 - 16 * 1024;     // (the kernel's static shared memory comes on top)
        if (smem > allowed) {
            cudaError_t e = cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "sample: %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
            allowed = smem;
        }
        cudaError_t e = launch_chained_cluster(sample_cluster_kernel, dim3(n_rows * SC), dim3(STC), smem, dim3(SC, 1, 1), stream,
                                               logits, ld, V, S, temperature, top_k, top_p, rng_key, rng_ctr, out_token,
                                               next_token, next_pos, row_slot);
        if (e != cudaSuccess) return vlrf_fail(VLRF_ERR_CUDA, "sample: %s", cudaGetErrorString(e));
        return vlrf_check_launch("sample");
    }
    launch_chained(sample_kernel, dim3(n_rows), dim3(ST), 0, stream, logits, ld, V, temperature, top_k, top_p, rng_key,
                   rng_ctr, out_token, next_token, next_pos, row_slot);
    return vlrf_check_launch("sample");
}

extern "C" int vlrf_apply_penalties(float* logits, int ld, int n_rows, int V, const int* gen, int gen_ld,
                                    const int* gen_len, const float* rep, const float* freq,
                                    const float* pres, const int* ngram, cudaStream_t stream) {
    VLRF_REQUIRE(n_rows >= 0 && V > 0 && ld >= V && gen_ld > 0, "penalties: bad sizes (the history needs a width)");
    if (n_rows == 0) return VLRF_OK;
    penalties_kernel<<<n_rows, 256, 0, stream>>>(logits, ld, V, gen, gen_ld, gen_len, rep, freq, pres, ngram);
    return vlrf_check_launch("penalties");
}
