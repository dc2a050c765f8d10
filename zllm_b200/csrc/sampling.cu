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
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(const float* __restrict__ logits,
                                                                const float* __restrict__ temps,
                                                                const unsigned* __restrict__ seeds,
                                                                int* __restrict__ out, int V) {
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
__global__ void __launch_bounds__(256) sample_chunks_kernel(const float* __restrict__ logits,
                                                            const float* __restrict__ temps,
                                                            const unsigned* __restrict__ seeds, int* __restrict__ out,
                                                            int V, float* __restrict__ part_v, int* __restrict__ part_i,
                                                            unsigned* __restrict__ counters) {
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
// entries leave (-3e38, -1) sentinels.
__global__ void __launch_bounds__(SAMPLE_THREADS) topk_kernel(const float* __restrict__ logits, float* __restrict__ vals,
                                                              int* __restrict__ idxs, int V, int k) {
    __shared__ float sv[32];
    __shared__ int si[32];
    __shared__ float win_v;
    __shared__ int win_i;
    const int row = blockIdx.x;
    const float* lg = logits + (size_t)row * V;
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int c = threadIdx.x; c < V; c += blockDim.x) {
            const float v = lg[c];
            const bool below = (v < prev_v) || (v == prev_v && c > prev_i);
            if (below && better(v, c, bv, bi)) { bv = v; bi = c; }
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
                vals[(size_t)row * k + r] = none ? -3.0e38f : bv;
                idxs[(size_t)row * k + r] = none ? -1 : bi;
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

ZLLM_API int zllm_topk(const float* logits, float* vals, int* idxs, int R, int V, int k, void* stream) {
    if (R <= 0) return 0;
    if (V <= 0 || k <= 0) return ZLLM_ERR_UNSUPPORTED;
    topk_kernel<<<R, SAMPLE_THREADS, 0, (cudaStream_t)stream>>>(logits, vals, idxs, V, k);
    return launch_status();
}

// After a decode step sampled ``out``: make the step's own inputs those of the next step, so
// that a captured decode graph can be replayed several times without the host in between.
// tok <- out, pos += 1, seed += 0x9E3779B1 (the per-token seed rule of
// zllm src/backend/gpu/sampling.rs:9); the sampled tokens are also appended to a history ring
// [hist_cap, B] that the host reads once at the end.  One block; B <= 1024.
__global__ void advance_decode_kernel(int* __restrict__ tok, int* __restrict__ pos, const int* __restrict__ row_slot,
                                      unsigned* __restrict__ seeds, const int* __restrict__ out,
                                      int* __restrict__ hist, int* __restrict__ counter, int hist_cap, int B) {
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
