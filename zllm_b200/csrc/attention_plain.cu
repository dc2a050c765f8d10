// Plain attention over the paged cache: one warp per (row, query head), every
// key of the row's request from its window's first to its own position, online
// softmax in float32, fixed order.
//
// The math of zllm's BDSDPA_PAGED (src/backend/gpu/shaders.rs:670-725): a row is
// (position, slot); keys are gathered through the block table; query head h
// reads kv head h / (nq/nkv); scores q.k * scale; running max m, running sum l,
// accumulator rescaled by exp(m_old - m_new).  There one thread walks the keys;
// here a warp takes 32 keys at a time, which fixes the order by the position
// alone: the result for a row does not depend on the batch it came in, on how
// its prompt was cut, or on which pages hold its keys.
//
// Used by the 32-bit path for every row, and by the bfloat16 path for head
// sizes the tensor-core kernels do not take.
#include "common.cuh"
#include <math.h>

#define MAX_HD 256

template <typename AT>
__global__ void __launch_bounds__(128) attention_plain_kernel(
    const AT* qkv, AT* out, const int* positions,
    const int* row_slot, const AT* k_pages, const AT* v_pages,
    const int* __restrict__ table, int max_blocks, int bs, int nq, int nkv, int hd, float scale, int window) {
    __shared__ float qs[4][MAX_HD];
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * 4 + warp;
    if (h >= nq) return;
    const int slot = row_slot[t];
    AT* o = out + ((size_t)t * nq + h) * hd;
    if (slot < 0) {
        for (int d = lane; d < hd; d += 32) o[d] = from_f32<AT>(0.f);
        return;
    }
    const int pos = positions[t];
    const int kvh = h / (nq / nkv);
    const AT* q = qkv + (size_t)t * (nq + 2 * nkv) * hd + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[warp][d] = to_f32(q[d]);
    __syncwarp();
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* trow = table + (size_t)slot * max_blocks;
    float m = -INFINITY, l = 0.f;
    float acc[MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;
    for (int base = lo; base <= pos; base += 32) {
        const int key = base + lane;
        const bool valid = key <= pos;
        long long off = -1;
        float s = -INFINITY;
        if (valid) {
            const int page = trow[key / bs];
            if (page >= 0) {
                off = (((long long)page * nkv + kvh) * bs + (key % bs)) * hd;
                const AT* k = k_pages + off;
                float dot = 0.f;
                for (int d = 0; d < hd; ++d) dot = fmaf(qs[warp][d], to_f32(k[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        const float corr = (m_new == -INFINITY) ? 1.f : expf(m - m_new);   // first chunk: m = -inf, exp(-inf) = 0
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= corr;
        const int n = min(32, pos - base + 1);
        for (int j = 0; j < n; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long oj = __shfl_sync(0xffffffffu, off, j);
            if (oj < 0) continue;
            const AT* v = v_pages + oj;
#pragma unroll
            for (int i = 0; i < MAX_HD / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < hd) acc[i] = fmaf(pj, to_f32(v[d]), acc[i]);
            }
        }
        m = m_new;
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) o[d] = from_f32<AT>(acc[i] * inv);
    }
}

ZLLM_API int zllm_attention_plain(const void* qkv, void* out, const int* positions, const int* row_slot,
                                  const void* k_pages, const void* v_pages, const int* table, int max_blocks, int bs,
                                  int T, int nq, int nkv, int hd, float scale, int window, int is_bf16, void* stream) {
    if (T <= 0) return 0;
    if (hd > MAX_HD || hd <= 0 || nkv <= 0 || nq % nkv) return ZLLM_ERR_UNSUPPORTED;
    dim3 grid(T, (nq + 3) / 4);
    cudaStream_t s = (cudaStream_t)stream;
    if (is_bf16)
        attention_plain_kernel<bf16><<<grid, 128, 0, s>>>((const bf16*)qkv, (bf16*)out, positions, row_slot,
                                                          (const bf16*)k_pages, (const bf16*)v_pages, table, max_blocks,
                                                          bs, nq, nkv, hd, scale, window);
    else
        attention_plain_kernel<float><<<grid, 128, 0, s>>>((const float*)qkv, (float*)out, positions, row_slot,
                                                           (const float*)k_pages, (const float*)v_pages, table,
                                                           max_blocks, bs, nq, nkv, hd, scale, window);
    return launch_status();
}
