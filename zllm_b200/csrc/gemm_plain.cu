// Plain product out = x W^T on CUDA cores, float32 accumulation, any sizes.
//
// This is the true 32-bit path's product and the catch-all for sizes the
// tensor-core kernels refuse.  Each output element is accumulated by ONE thread
// over k = 0..K-1 in that order, so the value of out[m][n] depends on row m of x
// and row n of W only -- never on how many rows the batch has, where the row
// sits in it, or what the other rows are.
//
// Epilogues (the reference folds the residual add into its O and down products
// with an `acc` flag, zllm src/backend/gpu/mod.rs:2492-2497, and concatenates
// gate and up into one weight, src/backend/vulkan/mod.rs:1141-1167):
//   MODE_STORE   out[m][n]  = acc                     (out dtype OT)
//   MODE_ADD     out[m][n] += acc                     (out float32: the residual)
//   MODE_SWIGLU  out[m][j]  = silu(gate_j) * up_j     W is [2I, K] with rows in
//                groups of 16: 8 gate rows, then the 8 up rows of the same j.
#include "common.cuh"

#define MODE_STORE 0
#define MODE_ADD 1
#define MODE_SWIGLU 2

#define BM 64
#define BN 64
#define BK 16

template <typename AT, typename OT, int MODE>
__global__ void __launch_bounds__(256) gemm_plain_kernel(const AT* x, const AT* __restrict__ w,
                                                         OT* out, int M, int N, int K) {
    // N counts output columns (for SWIGLU: the intermediate size I, W has 2I rows)
    __shared__ float xs[BK][BM + 1];
    __shared__ float ws[BK][BN + 1];
    __shared__ float us[MODE == MODE_SWIGLU ? BK : 1][BN + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;      // 16 x 16 threads, 4x4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[4][4] = {};
    float accu[MODE == MODE_SWIGLU ? 4 : 1][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int i = threadIdx.x; i < BM * BK; i += 256) {
            const int r = i / BK, c = i - r * BK;
            const int m = m0 + r, k = k0 + c;
            xs[c][r] = (m < M && k < K) ? to_f32(x[(size_t)m * K + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < BN * BK; i += 256) {
            const int r = i / BK, c = i - r * BK;
            const int n = n0 + r, k = k0 + c;
            if (MODE == MODE_SWIGLU) {
                const size_t grow = (size_t)(n >> 3) * 16 + (n & 7);
                ws[c][r] = (n < N && k < K) ? to_f32(w[grow * K + k]) : 0.f;
                us[c][r] = (n < N && k < K) ? to_f32(w[(grow + 8) * K + k]) : 0.f;
            } else {
                ws[c][r] = (n < N && k < K) ? to_f32(w[(size_t)n * K + k]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
            if (MODE == MODE_SWIGLU) {
#pragma unroll
                for (int j = 0; j < 4; ++j) u[j] = us[kk][tx * 4 + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
                    if (MODE == MODE_SWIGLU) accu[i][j] = fmaf(a[i], u[j], accu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            const size_t o = (size_t)m * N + n;
            if (MODE == MODE_STORE) out[o] = from_f32<OT>(acc[i][j]);
            else if (MODE == MODE_ADD) out[o] = from_f32<OT>(to_f32(out[o]) + acc[i][j]);
            else {
                const float g = acc[i][j];
                out[o] = from_f32<OT>(g / (1.f + expf(-g)) * accu[i][j]);
            }
        }
    }
}

template <typename AT, typename OT>
static int launch_plain(const void* x, const void* w, void* out, int M, int N, int K, int mode, cudaStream_t s) {
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (mode == MODE_STORE)
        gemm_plain_kernel<AT, OT, MODE_STORE><<<grid, 256, 0, s>>>((const AT*)x, (const AT*)w, (OT*)out, M, N, K);
    else if (mode == MODE_ADD)
        gemm_plain_kernel<AT, OT, MODE_ADD><<<grid, 256, 0, s>>>((const AT*)x, (const AT*)w, (OT*)out, M, N, K);
    else
        gemm_plain_kernel<AT, OT, MODE_SWIGLU><<<grid, 256, 0, s>>>((const AT*)x, (const AT*)w, (OT*)out, M, N, K);
    return launch_status();
}

// x [M,K], w [N,K] (SWIGLU: [2N,K]) both of dtype in_bf16 ? bf16 : float32; out [M,N] bf16 or float32.
ZLLM_API int zllm_gemm_plain(const void* x, const void* w, void* out, int M, int N, int K, int mode, int in_bf16,
                             int out_bf16, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || mode < 0 || mode > 2) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_ADD && out_bf16) return ZLLM_ERR_UNSUPPORTED;      // the residual stream is float32
    if (mode == MODE_SWIGLU && (N % 8)) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (in_bf16) {
        if (out_bf16) return launch_plain<bf16, bf16>(x, w, out, M, N, K, mode, s);
        return launch_plain<bf16, float>(x, w, out, M, N, K, mode, s);
    }
    if (out_bf16) return ZLLM_ERR_UNSUPPORTED;
    return launch_plain<float, float>(x, w, out, M, N, K, mode, s);
}
