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

// out[row][head][:] = sum_s O_s e^{m_s - M} / sum_s l_s e^{m_s - M} over the row's splits, in split order
template <int HD>
__global__ void decode_combine_kernel(const int* __restrict__ rows, const int* __restrict__ positions,
                                      const int* __restrict__ row_slot, const float* __restrict__ part_o,
                                      const float* __restrict__ part_ml, bf16* __restrict__ out, int nq, int window,
                                      int max_splits) {
    pdl_trigger();
    pdl_wait();
    const int row = rows[blockIdx.x];
    const int h = blockIdx.y;
    bf16* o = out + ((size_t)row * nq + h) * HD;
    if (row_slot[row] < 0) {
        for (int d = threadIdx.x; d < HD; d += blockDim.x) o[d] = __float2bfloat16_rn(0.f);
        return;
    }
    const int pos = positions[row];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int ns = (pos - lo) / SPLIT_KEYS + 1;
    const size_t base = ((size_t)blockIdx.x * nq + h) * max_splits;
    float M = -INFINITY;
    for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
    float L = 0.f;
    for (int s = 0; s < ns; ++s) {
        const float ms = part_ml[(base + s) * 2];
        L += part_ml[(base + s) * 2 + 1] * ((ms == -INFINITY) ? 0.f : exp2f(ms - M));
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float acc = 0.f;
        for (int s = 0; s < ns; ++s) {
            const float ms = part_ml[(base + s) * 2];
            acc += part_o[(base + s) * HD + d] * ((ms == -INFINITY) ? 0.f : exp2f(ms - M));
        }
        o[d] = __float2bfloat16_rn(acc * inv);
    }
}

