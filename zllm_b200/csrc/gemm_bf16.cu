// bfloat16 products on tensor cores for SMALL row counts (decode and short portions):
// out[m][n] = sum_k x[m][k] w[n][k], M <= 64, float32 accumulation.
//
// A decode step is bound by reading every weight once (zllm measures the same on its
// hardware: "decode matvec bandwidth ~84 % of peak", BENCHMARKS.md:29,122; its kernels
// for this regime are Q4K_SKINNY / Q4K_MATVEC, src/backend/gpu/shaders.rs:13-167).  So the
// weight matrix is the streamed operand: it is the M side of mma.sync.m16n8k16 (16 weight
// rows per warp) and is loaded straight from global memory into fragment registers with
// 16-byte loads; the few rows of x are the N side (8 per tile), staged in shared memory
// and shared by the CTA's 8 warps.  Because the order of k inside a tensor-core step is
// free as long as both operands agree, lane (g, t) simply takes the 16 consecutive k at
// k0 + 16 t of row g and g + 8 (four lanes cover 128 contiguous bytes of a row) and the same
// k of its x row -- no shuffles, no ldmatrix.
//
// To fill 148 SMs when N is small, K is split over a thread-block CLUSTER (1, 2, 4 or 8
// CTAs); the partial tiles are summed through distributed shared memory in rank order, so
// the result is deterministic and needs no scratch in global memory.  The split depends on
// (N, K) only; a column of the tile (a row of x) never mixes with another: the value of
// out[m][:] does not depend on what else is in the batch.
//
// Epilogues as in gemm_plain.cu: store (bf16 or float32), add into float32, swiglu on
// weights interleaved in groups of 8 gate rows + 8 up rows.
#include "common.cuh"
#include <cooperative_groups.h>
#include <cuda_pipeline.h>

namespace cg = cooperative_groups;

#define MODE_STORE 0
#define MODE_ADD 1
#define MODE_SWIGLU 2

#define SK_ROWS 128          // weight rows per CTA (8 warps x 16)
#define SK_KC 256            // k per shared-memory chunk of x
#define SK_XSTRIDE (SK_KC + 8)   // +16 bytes per row: conflict-free 16-byte reads

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                               unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

template <int NT>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                          void* __restrict__ out, int M, int N, int K, int kslice,
                                                          int mode, int out_bf16, int w_rows) {
    constexpr int MP = NT * 8;                       // padded rows of x
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* xs = reinterpret_cast<bf16*>(smem_raw);    // [2][MP][SK_XSTRIDE]
    float* red = reinterpret_cast<float*>(smem_raw); // [SK_ROWS][MP + 1], aliases xs after the main loop
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank();
    const int csize = (int)cluster.num_blocks();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * SK_ROWS;           // first weight row of the CTA
    const int ra = row0 + warp * 16 + g, rb = ra + 8;
    const bool va = ra < w_rows, vb = rb < w_rows;
    const bf16* wa = w + (size_t)(va ? ra : 0) * K;
    const bf16* wb = w + (size_t)(vb ? rb : 0) * K;
    const int k_begin = crank * kslice;
    const int k_end = min(K, k_begin + kslice);
    float acc[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;

    auto load_x_chunk = [&](int buf, int kc) {
        bf16* dst = xs + (size_t)buf * MP * SK_XSTRIDE;
        for (int i = threadIdx.x; i < MP * (SK_KC / 8); i += 256) {
            const int m = i / (SK_KC / 8), c = i - m * (SK_KC / 8);
            const int k = kc + c * 8;
            bf16* d = dst + (size_t)m * SK_XSTRIDE + c * 8;
            if (m < M && k < k_end) __pipeline_memcpy_async(d, x + (size_t)m * K + k, 16);
            else *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
        }
        __pipeline_commit();
    };

    const int n_chunks = (k_end > k_begin) ? (k_end - k_begin + SK_KC - 1) / SK_KC : 0;
    // weights of a chunk: 4 steps of 64 k, two 16-byte loads per row per step
    uint4 fa[4][2], fb[4][2];
    auto load_w_chunk = [&](int kc) {
#pragma unroll
        for (int s = 0; s < 4; ++s) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int k = kc + s * 64 + t * 16 + hf * 8;
                const bool in = k < k_end;
                fa[s][hf] = (va && in) ? ldg_stream(wa + k) : make_uint4(0, 0, 0, 0);
                fb[s][hf] = (vb && in) ? ldg_stream(wb + k) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    // Weights do not depend on the kernel before this one: let the next kernel start, fetch the
    // first chunk into registers and ask L2 for the rest of this CTA's slice, and only then wait
    // for x.
    pdl_trigger();
    if (n_chunks > 0) load_w_chunk(k_begin);
    for (int k = k_begin + SK_KC + t * 64; k < k_end; k += 256) {      // one 128-byte line per lane and row
        if (va) asm volatile("prefetch.global.L2 [%0];" ::"l"(wa + k));
        if (vb) asm volatile("prefetch.global.L2 [%0];" ::"l"(wb + k));
    }
    pdl_wait();
    if (n_chunks > 0) load_x_chunk(0, k_begin);
    for (int c = 0; c < n_chunks; ++c) {
        const int kc = k_begin + c * SK_KC;
        if (c > 0) load_w_chunk(kc);
        if (c + 1 < n_chunks) load_x_chunk((c + 1) & 1, kc + SK_KC);
        else __pipeline_commit();
        __pipeline_wait_prior(1);                    // chunk c of x has landed
        __syncthreads();
        const bf16* xb = xs + (size_t)(c & 1) * MP * SK_XSTRIDE;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const uint4 A = fa[s][hf], B = fb[s][hf];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    const uint4 X = *reinterpret_cast<const uint4*>(xb + (size_t)(nt * 8 + g) * SK_XSTRIDE + s * 64 +
                                                                    t * 16 + hf * 8);
                    mma_bf16_16816(acc[nt], A.x, B.x, A.y, B.y, X.x, X.y);
                    mma_bf16_16816(acc[nt], A.z, B.z, A.w, B.w, X.z, X.w);
                }
            }
        }
        __syncthreads();                             // everyone is done with buffer c & 1
    }
    __pipeline_wait_prior(0);
    __syncthreads();
    // partial tile -> shared memory [row][m]
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const int m = nt * 8 + 2 * t;
        float* r0 = red + (size_t)(warp * 16 + g) * (MP + 1) + m;
        float* r1 = red + (size_t)(warp * 16 + g + 8) * (MP + 1) + m;
        r0[0] = acc[nt][0]; r0[1] = acc[nt][1];
        r1[0] = acc[nt][2]; r1[1] = acc[nt][3];
    }
    cluster.sync();
    // each CTA of the cluster finishes SK_ROWS / csize rows: sum the partials in rank order
    const int rows_per = SK_ROWS / csize;
    const int rbase = crank * rows_per;
    const float* peer[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) peer[q] = q < csize ? cluster.map_shared_rank(red, q) : red;
    if (mode == MODE_SWIGLU) {
        const int outs_per = rows_per / 2;           // gate/up pairs
        const int I = N;
        for (int i = threadIdx.x; i < outs_per * M; i += 256) {
            const int m = i / outs_per, j = i - m * outs_per;
            const int grow = rbase + (j >> 3) * 16 + (j & 7);
            const int col = (row0 + rbase) / 2 + j;
            if (col >= I) continue;
            float gsum = 0.f, usum = 0.f;
            for (int q = 0; q < csize; ++q) {
                gsum += peer[q][(size_t)grow * (MP + 1) + m];
                usum += peer[q][(size_t)(grow + 8) * (MP + 1) + m];
            }
            const float v = gsum / (1.f + expf(-gsum)) * usum;
            if (out_bf16) reinterpret_cast<bf16*>(out)[(size_t)m * I + col] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(out)[(size_t)m * I + col] = v;
        }
    } else {
        for (int i = threadIdx.x; i < rows_per * M; i += 256) {
            const int m = i / rows_per, r = i - m * rows_per;
            const int n = row0 + rbase + r;
            if (n >= N) continue;
            float sum = 0.f;
            for (int q = 0; q < csize; ++q) sum += peer[q][(size_t)(rbase + r) * (MP + 1) + m];
            const size_t o = (size_t)m * N + n;
            if (mode == MODE_ADD) reinterpret_cast<float*>(out)[o] += sum;
            else if (out_bf16) reinterpret_cast<bf16*>(out)[o] = __float2bfloat16_rn(sum);
            else reinterpret_cast<float*>(out)[o] = sum;
        }
    }
    cluster.sync();                                  // peers may still be reading this CTA's partials
}

template <int NT>
static int launch_skinny(const void* x, const void* w, void* out, int M, int N, int K, int mode, int out_bf16,
                         cudaStream_t s) {
    const int w_rows = mode == MODE_SWIGLU ? 2 * N : N;
    const int tiles = (w_rows + SK_ROWS - 1) / SK_ROWS;
    // split K over a cluster until about two CTAs per SM exist; the choice depends on (N, K) only
    int csize = 1;
    while (csize < 8 && tiles * csize < 296 && K / (csize * 2) >= 256) csize *= 2;
    int kslice = ((K + csize - 1) / csize + 63) / 64 * 64;
    constexpr int MP = NT * 8;
    size_t smem = (size_t)2 * MP * SK_XSTRIDE * sizeof(bf16);
    const size_t red_bytes = (size_t)SK_ROWS * (MP + 1) * sizeof(float);
    if (red_bytes > smem) smem = red_bytes;
    auto kern = gemm_skinny_kernel<NT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, csize, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = csize;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, kern, (const bf16*)x, (const bf16*)w, out, M, N, K, kslice, mode, out_bf16, w_rows);
    return (int)e;
}

// x [M,K] bf16, w [N,K] bf16 ([2N,K] for swiglu), out [M,N] bf16 or float32.  M <= 64, K % 8 == 0.
ZLLM_API int zllm_gemm_skinny_bf16(const void* x, const void* w, void* out, int M, int N, int K, int mode,
                                   int out_bf16, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K % 8) || mode < 0 || mode > 2) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_ADD && out_bf16) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_SWIGLU && (N % 8)) return ZLLM_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return ZLLM_ERR_UNSUPPORTED;     // 16-byte loads
    cudaStream_t s = (cudaStream_t)stream;
    if (M <= 8) return launch_skinny<1>(x, w, out, M, N, K, mode, out_bf16, s);
    if (M <= 16) return launch_skinny<2>(x, w, out, M, N, K, mode, out_bf16, s);
    if (M <= 32) return launch_skinny<4>(x, w, out, M, N, K, mode, out_bf16, s);
    return launch_skinny<8>(x, w, out, M, N, K, mode, out_bf16, s);
}
