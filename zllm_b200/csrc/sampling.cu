// Sampling on the device, so that only token ids go back to the host.
//
// zllm's kernels (src/backend/gpu/shaders.rs): BARGMAX 758-789 (strict '>' keeps
// the lowest index), BSAMPLE 791-850 (Gumbel-max: argmax_i(logit_i/temp -
// log(-log u_i)), u_i = ((hash(seed ^ hash(i)) >> 8) + 0.5) / 2^24, temp <= 0 ->
// plain argmax), BTOPK 852-905 (K rounds of "largest strictly below the previous
// winner", value descending, index ascending).  Ties here ALWAYS resolve to the
// lowest index, also across threads (the reference's tree reduction keeps the
// lower thread, which is not always the lower index).
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ unsigned hash_u32(unsigned h) {
    h ^= h >> 16; h *= 0x7feb352du;
    h ^= h >> 15; h *= 0x846ca68bu;
    h ^= h >> 16;
    return h;
}
__device__ __forceinline__ float rand01(unsigned seed, unsigned i) {
    const unsigned r = hash_u32(seed ^ hash_u32(i));
    return ((float)(r >> 8) + 0.5f) / 16777216.0f;
}
__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
    return v > bv || (v == bv && i < bi);
}

#define SAMPLE_THREADS 1024

// one block per row; out[row] = sampled token
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* logits,
                                                                const float* temps,
                                                                const unsigned* seeds,
                                                                int* out, int V) {
    __shared__ float sv[32];
    __shared__ int si[32];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const float* lg = logits + (size_t)row * V;
    const float temp = temps ? temps[row] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float inv_t = greedy ? 1.f : 1.f / temp;
    const unsigned seed = seeds ? seeds[row] : 0u;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = threadIdx.x; k < V; k += blockDim.x) {
        float v = lg[k];
        if (!greedy) v = v * inv_t + (-logf(-logf(rand01(seed, (unsigned)k))));
        if (better(v, k, bv, bi)) { bv = v; bi = k; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (w == 0) {
        const int nw = blockDim.x >> 5;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[row] = (bi == 0x7fffffff) ? 0 : bi;   // all-NaN row: token 0
    }
}

// The same over a large vocabulary with many blocks per row: each block scans one chunk and
// writes its best (value, index); the block that arrives last for a row (a counter in global
// memory) picks the best of the chunks and resets the counter.  "Best" is the largest value,
// the lowest index among equals, which does not depend on the order of arrival.
#define SAMPLE_CHUNKS 64
__global__ void __launch_bounds__(256) sample_chunks_kernel(const float* logits,
                                                            const float* temps,
                                                            const unsigned* seeds, int* out,
                                                            int V, float* part_v, int* part_i,
                                                            unsigned* counters) {
    __shared__ float sv[8];
    __shared__ int si[8];
    __shared__ bool last;
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, chunk = blockIdx.y;
    const int per = (V + SAMPLE_CHUNKS - 1) / SAMPLE_CHUNKS;
    const int lo = chunk * per, hi = min(V, lo + per);
    const float* lg = logits + (size_t)row * V;
    const float temp = temps ? temps[row] : 0.f;
    const bool greedy = !(temp > 0.f);
    const float inv_t = greedy ? 1.f : 1.f / temp;
    const unsigned seed = seeds ? seeds[row] : 0u;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = lo + threadIdx.x; k < hi; k += blockDim.x) {
        float v = lg[k];
        if (!greedy) v = v * inv_t + (-logf(-logf(rand01(seed, (unsigned)k))));
        if (better(v, k, bv, bi)) { bv = v; bi = k; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    if (lane == 0) { sv[w] = bv; si[w] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int q = 1; q < 8; ++q)
            if (better(sv[q], si[q], bv, bi)) { bv = sv[q]; bi = si[q]; }
        part_v[(size_t)row * SAMPLE_CHUNKS + chunk] = bv;
        part_i[(size_t)row * SAMPLE_CHUNKS + chunk] = bi;
        __threadfence();
        last = atomicAdd(&counters[row], 1u) == SAMPLE_CHUNKS - 1;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    if (threadIdx.x < 32) {
        float v = -INFINITY;
        int i = 0x7fffffff;
        for (int c = threadIdx.x; c < SAMPLE_CHUNKS; c += 32) {
            const float cv = part_v[(size_t)row * SAMPLE_CHUNKS + c];
            const int ci = part_i[(size_t)row * SAMPLE_CHUNKS + c];
            if (better(cv, ci, v, i)) { v = cv; i = ci; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, i, o);
            if (better(ov, oi, v, i)) { v = ov; i = oi; }
        }
        if (threadIdx.x == 0) {
            out[row] = (i == 0x7fffffff) ? 0 : i;
            counters[row] = 0u;                      // ready for the next call
        }
    }
}

// scratch (may be null: one block per row then): part_v [R][64] float, part_i [R][64] int,
// counters [R] unsigned, all zero before the first call.
ZLLM_API int zllm_sample(const float* logits, const float* temps, const unsigned* seeds, int* out, int R, int V,
                         float* part_v, int* part_i, unsigned* counters, void* stream) {
    if (R <= 0) return 0;
    if (V <= 0) return ZLLM_ERR_UNSUPPORTED;
    if (part_v != nullptr && V >= 16384)
        return launch_pdl(sample_chunks_kernel, dim3(R, SAMPLE_CHUNKS), dim3(256), 0, (cudaStream_t)stream, logits, temps,
                          seeds, out, V, part_v, part_i, counters);
    return launch_pdl(sample_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, logits, temps, seeds, out, V);
}

// top-k candidates in descending order (value desc, index asc); fewer than k distinct
// entries leave (-3e38, -1) sentinels.  One block selects among ``count`` candidates of one row:
// K rounds of "the best strictly below the previous winner".  ``cidx`` == nullptr: candidate c is
// vocabulary entry first + c; else its vocabulary index is cidx[c] (-1: no candidate).

__device__ __forceinline__ void topk_select(const float* __restrict__ cv, const int* __restrict__ cidx, int first, int count,
                                            float* __restrict__ vals, int* __restrict__ idxs, int k) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float win_v;
    __shared__ int win_i;
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int c = threadIdx.x; c < count; c += blockDim.x) {
            const int gi = cidx ? cidx[c] : first + c;
            if (gi < 0) continue;
            const float v = cv[c];
            const bool below = (v < prev_v) || (v == prev_v && gi > prev_i);
            if (below && better(v, gi, bv, bi)) { bv = v; bi = gi; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
        }
        const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
        if (lane == 0) { sv[w] = bv; si[w] = bi; }
        __syncthreads();
        if (w == 0) {
            const int nw = blockDim.x >> 5;
            bv = lane < nw ? sv[lane] : -INFINITY;
            bi = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi, bv, bi)) { bv = ov; bi = oi; }
            }
            if (lane == 0) {
                const bool none = (bi == 0x7fffffff);
                vals[r] = none ? -3.0e38f : bv;
                idxs[r] = none ? -1 : bi;
                win_v = none ? -INFINITY : bv;
                win_i = none ? 0x7fffffff : bi;
            }
        }
        __syncthreads();
        prev_v = win_v;
        prev_i = win_i;
        __syncthreads();
    }
}

// the whole row in one block (any number of rows)
__global__ void __launch_bounds__(SAMPLE_THREADS) topk_kernel(const float* logits, float* vals,
                                                              int* idxs, int V, int k) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    topk_select(logits + (size_t)row * V, nullptr, 0, V, vals + (size_t)row * k, idxs + (size_t)row * k, k);
}
// Large vocabularies: selection by WARPS, without block barriers, and only among entries that can
// be among the k best.  (1) the row is cut into 64 groups; the smallest of the 64 group maxima is a
// floor: at least 64 entries are >= it, so nothing below it is among the 64 best.  (2) every one
// of 256 stretches of the row is reduced by one warp to its entries >= the floor, best first (a
// warp holds 32 x TOPK_E candidates in registers and runs rounds of "the largest key strictly
// below the previous winner" with shuffles only; it stops at the floor).  (3) the stretches' lists
// are merged the same way, 256 -> 32 -> 4 -> 1 lists.  The result is the k best of the row in the
// order of the one-block kernel.  k <= 64, 16384 <= V <= 131072.
#define TOPK_E 16                       // candidates per lane
#define TOPK_WARP_SPAN (32 * TOPK_E)    // candidates per warp
#define TOPK_STRETCHES 256              // stretches (warps) per row in step (2)
#define TOPK_GROUPS 64

// A candidate as one 64-bit key that orders like (value descending, index ascending): the float's
// bits made monotonic in the high word, the inverted index in the low word; 0 = no candidate.
__device__ __forceinline__ unsigned topk_mono(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ unsigned long long topk_key(float v, int i) {
    return ((unsigned long long)topk_mono(v) << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
}
__device__ __forceinline__ float topk_key_value(unsigned long long k) {
    const unsigned m = (unsigned)(k >> 32);
    return __uint_as_float((m & 0x80000000u) ? (m & 0x7FFFFFFFu) : ~m);
}
// Rounds over this lane's TOPK_E candidates (value cv[e], vocabulary index ci[e], -1: none) until k
// winners are out, none is left, or the next one lies below ``floor_m`` (monotonic bits of the floor;
// 0: no floor).  vals[0..k), idxs[0..k) get the winners, then (-3e38, -1).
__device__ __forceinline__ void warp_topk(const float (&cv)[TOPK_E], const int (&ci)[TOPK_E], float* __restrict__ vals,
                                          int* __restrict__ idxs, int k, unsigned floor_m) {
    const int lane = threadIdx.x & 31;
    for (int r = lane; r < k; r += 32) { vals[r] = -3.0e38f; idxs[r] = -1; }
    __syncwarp();
    unsigned long long key[TOPK_E];
#pragma unroll
    for (int e = 0; e < TOPK_E; ++e) key[e] = ci[e] >= 0 ? topk_key(cv[e], ci[e]) : 0ull;
    unsigned long long prev = ~0ull;
    for (int r = 0; r < k; ++r) {
        unsigned long long m[TOPK_E];
#pragma unroll
        for (int e = 0; e < TOPK_E; ++e) m[e] = key[e] < prev ? key[e] : 0ull;
#pragma unroll
        for (int w = TOPK_E / 2; w > 0; w >>= 1)
#pragma unroll
            for (int e = 0; e < w; ++e) m[e] = m[e] > m[e + w] ? m[e] : m[e + w];
        unsigned long long best = m[0];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, o);
            best = other > best ? other : best;
        }
        if (best == 0ull || (unsigned)(best >> 32) < floor_m) break;     // warp-uniform
        if (lane == 0) {
            vals[r] = topk_key_value(best);
            idxs[r] = (int)(0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFull));
        }
        prev = best;
    }
}

// (1) grid (R, TOPK_GROUPS): the maximum of each group of the row
__global__ void __launch_bounds__(256) topk_groupmax_kernel(const float* logits, float* gmax, int V) {
    __shared__ float sm[8];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, grp = blockIdx.y;
    const int len = (V + TOPK_GROUPS - 1) / TOPK_GROUPS;
    const int first = grp * len, last = min(V, first + len);
    const float* lg = logits + (size_t)row * V;
    float m = -INFINITY;
    for (int c = first + threadIdx.x; c < last; c += blockDim.x) m = fmaxf(m, lg[c]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w) m = fmaxf(m, sm[w]);
        gmax[(size_t)row * TOPK_GROUPS + grp] = m;
    }
}
// (2) grid (R, TOPK_STRETCHES / 8), 8 warps per block, a stretch per warp
__global__ void __launch_bounds__(256) topk_stretch_kernel(const float* logits, const float* gmax,
                                                           float* cand_v, int* cand_i, int V, int k) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float fl = fminf(gmax[(size_t)row * TOPK_GROUPS + lane], gmax[(size_t)row * TOPK_GROUPS + 32 + lane]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) fl = fminf(fl, __shfl_xor_sync(0xffffffffu, fl, o));
    const int stretch = blockIdx.y * 8 + warp;
    const int first = stretch * TOPK_WARP_SPAN;
    const float* lg = logits + (size_t)row * V;
    float cv[TOPK_E];
    int ci[TOPK_E];
#pragma unroll
    for (int e = 0; e < TOPK_E; ++e) {
        const int c = first + e * 32 + lane;
        ci[e] = c < V ? c : -1;
        cv[e] = c < V ? lg[c] : 0.f;
    }
    const size_t o = ((size_t)row * TOPK_STRETCHES + stretch) * k;
    warp_topk(cv, ci, cand_v + o, cand_i + o, k, topk_mono(fl));
}
// (3a) grid (R, 4), 8 warps per block: 256 lists -> 32 lists, a warp takes 8 lists (8 k <= 512 slots)
__global__ void __launch_bounds__(256) topk_merge1_kernel(const float* cand_v, const int* cand_i,
                                                          float* m1_v, int* m1_i, int k) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, warp = blockIdx.y * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const size_t src = ((size_t)row * TOPK_STRETCHES + warp * 8) * k;
    float cv[TOPK_E];
    int ci[TOPK_E];
#pragma unroll
    for (int e = 0; e < TOPK_E; ++e) {
        const int c = e * 32 + lane;
        const bool ok = c < 8 * k;
        ci[e] = ok ? cand_i[src + c] : -1;
        cv[e] = ok ? cand_v[src + c] : 0.f;
    }
    const size_t dst = ((size_t)row * 32 + warp) * k;
    warp_topk(cv, ci, m1_v + dst, m1_i + dst, k, 0u);
}
// (3b) grid (R), 4 warps: 32 lists -> 4 lists -> the row's k best
__global__ void __launch_bounds__(128) topk_merge2_kernel(const float* m1_v, const int* m1_i,
                                                          float* vals, int* idxs, int k) {
    __shared__ float tv[4 * 64];
    __shared__ int ti[4 * 64];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t src = ((size_t)row * 32 + warp * 8) * k;
    float cv[TOPK_E];
    int ci[TOPK_E];
#pragma unroll
    for (int e = 0; e < TOPK_E; ++e) {
        const int c = e * 32 + lane;
        const bool ok = c < 8 * k;
        ci[e] = ok ? m1_i[src + c] : -1;
        cv[e] = ok ? m1_v[src + c] : 0.f;
    }
    warp_topk(cv, ci, tv + warp * k, ti + warp * k, k, 0u);
    __syncthreads();
    if (warp == 0) {
#pragma unroll
        for (int e = 0; e < TOPK_E; ++e) {
            const int c = e * 32 + lane;
            const bool ok = c < 4 * k;
            ci[e] = ok ? ti[c] : -1;
            cv[e] = ok ? tv[c] : 0.f;
        }
        warp_topk(cv, ci, vals + (size_t)row * k, idxs + (size_t)row * k, k, 0u);
    }
}

// cand_v / cand_i: scratch of R x (TOPK_STRETCHES + 32) x k + R x TOPK_GROUPS entries each, or nullptr
// (one block per row).
ZLLM_API int zllm_topk(const float* logits, float* vals, int* idxs, int R, int V, int k, float* cand_v, int* cand_i,
                       void* stream) {
    if (R <= 0) return 0;
    if (V <= 0 || k <= 0) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (cand_v != nullptr && cand_i != nullptr && V >= 16384 && V <= TOPK_STRETCHES * TOPK_WARP_SPAN && k <= 64) {
        float* m1_v = cand_v + (size_t)R * TOPK_STRETCHES * k;
        int* m1_i = cand_i + (size_t)R * TOPK_STRETCHES * k;
        float* gmax = m1_v + (size_t)R * 32 * k;
        int rc = launch_pdl(topk_groupmax_kernel, dim3(R, TOPK_GROUPS), dim3(256), 0, s, logits, gmax, V);
        if (rc) return rc;
        rc = launch_pdl(topk_stretch_kernel, dim3(R, TOPK_STRETCHES / 8), dim3(256), 0, s, logits, (const float*)gmax, cand_v,
                        cand_i, V, k);
        if (rc) return rc;
        rc = launch_pdl(topk_merge1_kernel, dim3(R, 4), dim3(256), 0, s, (const float*)cand_v, (const int*)cand_i, m1_v, m1_i, k);
        if (rc) return rc;
        return launch_pdl(topk_merge2_kernel, dim3(R), dim3(128), 0, s, (const float*)m1_v, (const int*)m1_i, vals, idxs, k);
    }
    return launch_pdl(topk_kernel, dim3(R), dim3(SAMPLE_THREADS), 0, s, logits, vals, idxs, V, k);
}

// The draw among a row's descending candidates that zllm makes on the host
// (src/backend/gpu/sampling.rs:35-56), on the device and in double precision, so that a decode
// step with top-k / top-p sampling needs no host in between: probabilities exp((v - max) / T) of
// the first min(top_k, valid) candidates, normalised; cut where the cumulative mass reaches
// top_p; u from splitmix64(seed) (sampling.rs:24-30); inverse CDF.  Rows with ptemp <= 0 keep
// what ``out`` already holds (they were sampled by the argmax / Gumbel kernel).
__device__ __forceinline__ double splitmix01(unsigned seed) {
    unsigned long long z = (unsigned long long)seed * 0x9E3779B97F4A7C15ull + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return ((double)(z >> 40) + 0.5) / 16777216.0;
}
__global__ void pool_draw_kernel(const float* vals, const int* idxs, const double* ptemp,
                                 const int* topk, const double* topp,
                                 const unsigned* seeds, int* out, int k) {
    __shared__ double probs[64];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const double T = ptemp[row];
    if (!(T > 0.0)) return;
    const float* v = vals + (size_t)row * k;
    const int* ix = idxs + (size_t)row * k;
    int n = 0;
    while (n < k && v[n] > -3.0e37f) ++n;                  // (every thread counts: k <= 64)
    if (n == 0) { if (threadIdx.x == 0) out[row] = ix[0]; return; }
    const int tk = topk[row];
    const int kk = tk == 0 ? n : min(tk, n);
    const double mx = (double)v[0];
    for (int i = threadIdx.x; i < kk; i += blockDim.x) probs[i] = exp(((double)v[i] - mx) / T);
    __syncthreads();
    if (threadIdx.x != 0) return;
    double z = 0.0;
    for (int i = 0; i < kk; ++i) z += probs[i];
    for (int i = 0; i < kk; ++i) probs[i] = probs[i] / z;
    int cut = kk;
    const double tp = topp[row];
    if (tp > 0.0 && tp < 1.0) {
        double cum = 0.0;
        for (int i = 0; i < kk; ++i) {
            cum += probs[i];
            if (cum >= tp) { cut = i + 1; break; }
        }
    }
    double zc = 0.0;
    for (int i = 0; i < cut; ++i) zc += probs[i];
    const double target = splitmix01(seeds[row]) * zc;
    double acc = 0.0;
    int pick = ix[cut - 1];
    for (int i = 0; i < cut; ++i) {
        acc += probs[i];
        if (acc >= target) { pick = ix[i]; break; }
    }
    out[row] = pick;
}

// k <= 64
ZLLM_API int zllm_pool_draw(const float* vals, const int* idxs, const double* ptemp, const int* topk, const double* topp,
                            const unsigned* seeds, int* out, int R, int k, void* stream) {
    if (R <= 0) return 0;
    if (k <= 0 || k > 64) return ZLLM_ERR_UNSUPPORTED;
    return launch_pdl(pool_draw_kernel, dim3(R), dim3(64), 0, (cudaStream_t)stream, vals, idxs, ptemp, topk, topp, seeds, out, k);
}

// After a decode step sampled ``out``: make the step's own inputs those of the next step, so
// that a captured decode graph can be replayed several times without the host in between.
// tok <- out, pos += 1, seed += 0x9E3779B1 (the per-token seed rule of
// zllm src/backend/gpu/sampling.rs:9); the sampled tokens are also appended to a history ring
// [hist_cap, B] that the host reads once at the end.  One block; B <= 1024.
__global__ void advance_decode_kernel(int* tok, int* pos, const int* row_slot,
                                      unsigned* seeds, const int* out,
                                      int* hist, int* counter, int hist_cap, int B) {
    pdl_trigger();
    pdl_wait();
    const int r = threadIdx.x;
    const int c = counter[0];
    if (r < B) {
        const int t = out[r];
        if (row_slot[r] >= 0) {
            tok[r] = t;
            pos[r] += 1;
            seeds[r] += 0x9E3779B1u;
        }
        hist[(size_t)(c % hist_cap) * B + r] = t;
    }
    __syncthreads();
    if (r == 0) counter[0] = c + 1;
}

ZLLM_API int zllm_advance_decode(int* tok, int* pos, const int* row_slot, unsigned* seeds, const int* out, int* hist,
                                 int* counter, int hist_cap, int B, void* stream) {
    if (B <= 0) return 0;
    if (B > 1024 || hist_cap <= 0) return ZLLM_ERR_UNSUPPORTED;
    return launch_pdl(advance_decode_kernel, dim3(1), dim3(((B + 31) / 32) * 32), 0, (cudaStream_t)stream, tok, pos,
                      row_slot, seeds, out, hist, counter, hist_cap, B);
}
