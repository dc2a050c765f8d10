// Shared by the attention kernels: tile sizes, tensor-core and special-function helpers, and
// the kernel that merges the decode splits.
#pragma once
#include "common.cuh"
#include <math.h>

#define SPLIT_KEYS 256
#define DEC_WARPS 4
#define DEC_BLOCK 32            // keys per warp iteration in the decode kernel
#define PF_QROWS 128            // query rows per prefill CTA (= QUERY_TILE of the host's tile list)
#define PF_KEYS 64              // keys per prefill tile
#define PF_STAGES 3             // shared-memory tiles in flight

__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned a = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
// 2^x on the special-function unit (float32 in, float32 out; 2^-inf = 0)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// out[row][head][:] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the row's splits.
// One block per (row, head).  A long context has hundreds of splits (256 at 65,536 positions) and
// few rows, so the splits are spread over the block: for M and the denominator every thread
// takes every blockDim-th split, for the numerator the block is G = blockDim / HD groups of HD
// threads and group g takes the splits s = g, g + G, ...; the groups' sums are added in group
// order.  The order of every sum is fixed by the number of splits and the block's size NTHR:
// one group (the smallest block that covers HD) when the grid has at most 8 splits, else
// COMBINE_THREADS; the launcher chooses from the grid's split count alone (launch_combine).
#define COMBINE_THREADS 256
template <int HD, int NTHR>
__global__ void __launch_bounds__(NTHR) decode_combine_kernel(
    const int* rows, const int* positions, const int* row_slot,
    const float* part_o, const float* part_ml, bf16* out, int nq, int window,
    int max_splits, int n_splits) {
    constexpr int nthr = NTHR, G = NTHR / HD;                // groups of HD threads (at least one)
    __shared__ float s_red[NTHR / 32];
    __shared__ float s_acc[NTHR];
    pdl_trigger();
    const int row = rows[blockIdx.x];                        // inputs of the step: read before the wait
    const int slot_of_row = row_slot[row];
    const int pos = positions[row];
    pdl_wait();
    const int h = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    bf16* o = out + ((size_t)row * nq + h) * HD;
    if (slot_of_row < 0) {
        for (int d = tid; d < HD; d += nthr) o[d] = __float2bfloat16_rn(0.f);
        return;
    }
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    // never beyond what the split kernel's grid wrote (a caller that passed too few splits for
    // this row gets the keys of the splits it asked for, not someone else's partials)
    const int ns = min((pos - lo) / SPLIT_KEYS + 1, n_splits);
    const size_t base = ((size_t)blockIdx.x * nq + h) * max_splits;
    // M: the largest of the splits' maxima
    float m = -INFINITY;
    for (int s = tid; s < ns; s += nthr) m = fmaxf(m, part_ml[(base + s) * 2]);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    if (lane == 0) s_red[warp] = m;
    __syncthreads();
    float M = s_red[0];
#pragma unroll
    for (int w = 1; w < nthr / 32; ++w) M = fmaxf(M, s_red[w]);
    __syncthreads();
    // L: the denominator
    float l = 0.f;
    for (int s = tid; s < ns; s += nthr) {
        const float ms = part_ml[(base + s) * 2];
        l += part_ml[(base + s) * 2 + 1] * ((ms == -INFINITY) ? 0.f : exp2f(ms - M));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    if (lane == 0) s_red[warp] = l;
    __syncthreads();
    float L = 0.f;
#pragma unroll
    for (int w = 0; w < nthr / 32; ++w) L += s_red[w];
    const float inv = L > 0.f ? 1.f / L : 0.f;
    // the numerator: group g sums its splits for dim d
    const int g = tid / HD, d = tid - g * HD;
    if (g < G) {
        float acc = 0.f;
#pragma unroll 4
        for (int s = g; s < ns; s += G) {
            const float ms = part_ml[(base + s) * 2];
            acc += part_o[(base + s) * HD + d] * ((ms == -INFINITY) ? 0.f : exp2f(ms - M));
        }
        s_acc[g * HD + d] = acc;
    }
    __syncthreads();
    if (tid < HD) {
        float acc = 0.f;
#pragma unroll
        for (int gg = 0; gg < G; ++gg) acc += s_acc[gg * HD + tid];
        o[tid] = __float2bfloat16_rn(acc * inv);
    }
}

// The same merge by ONE WARP per (row, head): lane s holds split s's maximum and denominator, every
// lane takes HD / 32 dims and requests the numerators of the first 16 splits BEFORE anything waits
// for the maxima, so the kernel is one round trip to L2 and a few shuffles, with no block-wide
// barrier (with the loads inside the loop over the splits it was slower than the block kernel: a
// round trip per four splits; as it is, the batch-8 step went from 0.988 to 0.975 ms and batch 64
// from 24.0 k to 24.8 k tok/s).  The numerator is summed in split order, M and the denominator over
// a fixed shuffle tree.  Eight warps per block.
// Up to 32 splits (contexts up to 8,192) in one pass (FINAL).  Up to 1,024 splits in two: a first
// pass (not FINAL) merges every group of 32 splits into one partial of the same form (maximum,
// denominator, numerators), written to the slots [slot_out, ..) that the caller left free behind
// the row's own; the second pass merges those.  A row of 512 splits (131,000 positions) took the
// block kernel 35 us, a third of such a step.
#define COMBINE_WARP_MAX_SPLITS 32
// Two passes pay from a few hundred splits on (batch 1: 131,000 positions 1.93 -> 1.64 ms, 65,536
// 1.35 -> 1.31 ms; at 16,384 positions, 64 splits, two launches cost more than the block kernel:
// 0.85 -> 0.93 ms).
#define COMBINE_TWO_PASS_MIN_SPLITS 256
template <int HD, bool FINAL>
__global__ void __launch_bounds__(256) decode_combine_warp_kernel(
    const int* rows, const int* positions, const int* row_slot,
    float* part_o, float* part_ml, bf16* out, int nq, int window,
    int max_splits, int n_splits, int n_pairs, int slot_in, int level_div, int n_groups, int slot_out) {
    constexpr int DPL = (HD + 31) / 32;                      // dims per lane
    // which row, its slot and its position are inputs of the step (no kernel of the step writes
    // them): read before the wait, two dependent round trips that then cost nothing
    pdl_trigger();
    const int lane = threadIdx.x & 31;
    const int item = blockIdx.x * 8 + (threadIdx.x >> 5);    // (row index, head, group of 32 inputs)
    const bool live = item < n_pairs * n_groups;
    const int pair = live ? item / n_groups : 0, grp = item - pair * n_groups;
    const int ri = pair / nq, h = pair - ri * nq;
    const int row = rows[ri];
    const int slot_of_row = row_slot[row];
    const int pos = positions[row];
    pdl_wait();
    if (!live) return;
    bf16* o = out + ((size_t)row * nq + h) * HD;
    if (slot_of_row < 0) {
        if (FINAL) {
#pragma unroll
            for (int j = 0; j < DPL; ++j)
                if (lane + 32 * j < HD) o[lane + 32 * j] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int ns_row = min((pos - lo) / SPLIT_KEYS + 1, n_splits);       // the row's splits
    const int ns_in = (ns_row + level_div - 1) / level_div;              // inputs of this pass
    const int first = grp * 32;
    const int ns = min(32, ns_in - first);                               // inputs of this warp
    if (ns <= 0) return;                                                 // (not FINAL: a group beyond the row's splits)
    const size_t base = ((size_t)ri * nq + h) * max_splits + slot_in + first;
    // the numerators of the first 16 inputs are requested before anything waits for M
    float ov[16][DPL];
#pragma unroll
    for (int s = 0; s < 16; ++s)
#pragma unroll
        for (int j = 0; j < DPL; ++j)
            ov[s][j] = (s < ns && lane + 32 * j < HD) ? __ldcg(part_o + (base + s) * HD + lane + 32 * j) : 0.f;
    const float2 ml = lane < ns ? __ldcg(reinterpret_cast<const float2*>(part_ml + (base + lane) * 2)) : make_float2(-INFINITY, 0.f);
    float M = ml.x;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float f = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - M);
    float L = ml.y * f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    float acc[DPL];
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[j] = 0.f;
#pragma unroll
    for (int s = 0; s < 16; ++s) {
        const float fs = __shfl_sync(0xffffffffu, f, s);
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[j] += ov[s][j] * fs;      // inputs beyond ns: 0 x 0
    }
    for (int s = 16; s < ns; ++s) {
        const float fs = __shfl_sync(0xffffffffu, f, s);
#pragma unroll
        for (int j = 0; j < DPL; ++j)
            if (lane + 32 * j < HD) acc[j] += __ldcg(part_o + (base + s) * HD + lane + 32 * j) * fs;
    }
    if (FINAL) {
        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
        for (int j = 0; j < DPL; ++j)
            if (lane + 32 * j < HD) o[lane + 32 * j] = __float2bfloat16_rn(acc[j] * inv);
    } else {
        const size_t dst = ((size_t)ri * nq + h) * max_splits + slot_out + grp;
#pragma unroll
        for (int j = 0; j < DPL; ++j)
            if (lane + 32 * j < HD) part_o[dst * HD + lane + 32 * j] = acc[j];
        if (lane == 0) { part_ml[dst * 2] = M; part_ml[dst * 2 + 1] = L; }
    }
}

// The merge after a decode kernel with ``n_splits`` splits in its grid (programmatic dependent launch).
template <int HD>
static int launch_combine(int n_rows, int nq, int n_splits, cudaStream_t s, const int* rows, const int* positions,
                          const int* row_slot, const float* part_o, const float* part_ml, bf16* out, int window,
                          int max_splits) {
    constexpr int ONE = HD <= 32 ? 32 : (HD <= 64 ? 64 : 128);
    const int n_pairs = n_rows * nq;
    if (n_splits <= COMBINE_WARP_MAX_SPLITS)
        return launch_pdl(decode_combine_warp_kernel<HD, true>, dim3((n_pairs + 7) / 8), dim3(256), 0, s, rows, positions, row_slot,
                          (float*)part_o, (float*)part_ml, out, nq, window, max_splits, n_splits, n_pairs, 0, 1, 1, 0);
    const int n_groups = (n_splits + COMBINE_WARP_MAX_SPLITS - 1) / COMBINE_WARP_MAX_SPLITS;
    if (n_splits >= COMBINE_TWO_PASS_MIN_SPLITS && n_groups <= COMBINE_WARP_MAX_SPLITS && n_splits + n_groups <= max_splits) {
        // two passes; the groups' partials go to the free slots behind the grid's own
        int rc = launch_pdl(decode_combine_warp_kernel<HD, false>, dim3((n_pairs * n_groups + 7) / 8), dim3(256), 0, s, rows,
                            positions, row_slot, (float*)part_o, (float*)part_ml, out, nq, window, max_splits, n_splits, n_pairs, 0,
                            1, n_groups, n_splits);
        if (rc) return rc;
        return launch_pdl(decode_combine_warp_kernel<HD, true>, dim3((n_pairs + 7) / 8), dim3(256), 0, s, rows, positions, row_slot,
                          (float*)part_o, (float*)part_ml, out, nq, window, max_splits, n_splits, n_pairs, n_splits,
                          COMBINE_WARP_MAX_SPLITS, 1, 0);
    }
    if (n_splits <= 8)
        return launch_pdl(decode_combine_kernel<HD, ONE>, dim3(n_rows, nq), dim3(ONE), 0, s, rows, positions, row_slot, part_o,
                          part_ml, out, nq, window, max_splits, n_splits);
    return launch_pdl(decode_combine_kernel<HD, COMBINE_THREADS>, dim3(n_rows, nq), dim3(COMBINE_THREADS), 0, s, rows, positions,
                      row_slot, part_o, part_ml, out, nq, window, max_splits, n_splits);
}
