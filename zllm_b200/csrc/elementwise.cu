// Row-wise kernels: embedding gather, RMSNorm, SiLU-mul, row gather, rotary
// encoding fused with the write of keys and values into cache pages.
//
// Counterparts in zllm (WGSL, src/backend/gpu/shaders.rs): BNORM 545-564, BROPE
// 566-587, BKV_PACK 727-756, SILU_MUL 976-990; the embedding gather is done on
// the host there (src/backend/gpu/mod.rs:2450-2458).  The fusion of rotation and
// cache write follows its Vulkan path (decode_matvec_q4k_rope.comp).
// All sums, roots and rotations are float32 whatever the activation dtype.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
template <typename WT>
__global__ void embedding_kernel(const int* tok, const WT* __restrict__ table, float* out,
                                 int H, int V) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = tok[t];
    float* o = out + (size_t)t * H;
    if (id < 0 || id >= V) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const WT* row = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_f32(row[i]);
}

ZLLM_API int zllm_embedding(const int* tok, const void* table, float* out, int T, int H, int V, int table_bf16,
                            void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (table_bf16) return launch_pdl(embedding_kernel<bf16>, dim3(T), dim3(256), 0, s, tok, (const bf16*)table, out, H, V);
    return launch_pdl(embedding_kernel<float>, dim3(T), dim3(256), 0, s, tok, (const float*)table, out, H, V);
}

// ---------------------------------------------------------------- rmsnorm
// y = x * rsqrt(mean(x^2) + eps) * w ; x float32 [T,H]; w float32 or bf16; y AT.
// ``rows`` (may be null): y[t] is the norm of x[rows[t]] -- the rows whose logits are wanted go
// from the residual straight to the head's input, without a copy of their own.  The index list is
// an input of the step (no kernel writes it), so it is read before the wait.
template <typename WT, typename OT>
__global__ void rmsnorm_kernel(const float* x, const int* __restrict__ rows, const WT* __restrict__ w, OT* y, int H,
                               float eps) {
    __shared__ float red[33];
    pdl_trigger();
    const int src = rows != nullptr ? rows[blockIdx.x] : (int)blockIdx.x;
    pdl_wait();
    const float* xr = x + (size_t)src * H;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) { float v = xr[i]; ss += v * v; }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    OT* yr = y + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = from_f32<OT>(xr[i] * inv * to_f32(w[i]));
}

// The same with 16-byte loads and the row kept in registers (H % 4 == 0, H <= 256 * 4 * RV).
template <typename WT, typename OT, int RV>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const float* x, const int* __restrict__ rows,
                                                          const WT* __restrict__ w, OT* y, int H, float eps) {
    __shared__ float red[33];
    pdl_trigger();
    const int src = rows != nullptr ? rows[blockIdx.x] : (int)blockIdx.x;
    const int n4 = H >> 2;
    // the norm's weights are fetched before the wait (no kernel writes them): after it only x is read
    float wv[RV][4];
#pragma unroll
    for (int r = 0; r < RV; ++r) {
        const int i = threadIdx.x + r * 256;
#pragma unroll
        for (int e = 0; e < 4; ++e) wv[r][e] = i < n4 ? to_f32(w[4 * i + e]) : 0.f;
    }
    pdl_wait();
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)src * H);
    float4 v[RV];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < RV; ++r) {
        const int i = threadIdx.x + r * 256;
        v[r] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss += v[r].x * v[r].x + v[r].y * v[r].y + v[r].z * v[r].z + v[r].w * v[r].w;
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
    OT* yr = y + (size_t)blockIdx.x * H;
#pragma unroll
    for (int r = 0; r < RV; ++r) {
        const int i = threadIdx.x + r * 256;
        if (i >= n4) continue;
        const float o0 = v[r].x * inv * wv[r][0], o1 = v[r].y * inv * wv[r][1];
        const float o2 = v[r].z * inv * wv[r][2], o3 = v[r].w * inv * wv[r][3];
        if (sizeof(OT) == 2) {
            __nv_bfloat162 a = __floats2bfloat162_rn(o0, o1), b = __floats2bfloat162_rn(o2, o3);
            uint2 pk;
            pk.x = *reinterpret_cast<unsigned*>(&a);
            pk.y = *reinterpret_cast<unsigned*>(&b);
            *reinterpret_cast<uint2*>(yr + 4 * i) = pk;
        } else {
            *reinterpret_cast<float4*>(yr + 4 * i) = make_float4(o0, o1, o2, o3);
        }
    }
}

template <typename WT, typename OT>
static int launch_rmsnorm(const float* x, const int* rows, const void* w, void* y, int T, int H, float eps, cudaStream_t s) {
    const bool vec = (H % 4 == 0) && (((uintptr_t)x | (uintptr_t)y) % 16 == 0);
    if (vec && H <= 256 * 4 * 2)
        return launch_pdl(rmsnorm_vec_kernel<WT, OT, 2>, dim3(T), dim3(256), 0, s, x, rows, (const WT*)w, (OT*)y, H, eps);
    if (vec && H <= 256 * 4 * 8)
        return launch_pdl(rmsnorm_vec_kernel<WT, OT, 8>, dim3(T), dim3(256), 0, s, x, rows, (const WT*)w, (OT*)y, H, eps);
    const int th = H >= 1024 ? 256 : 128;
    return launch_pdl(rmsnorm_kernel<WT, OT>, dim3(T), dim3(th), 0, s, x, rows, (const WT*)w, (OT*)y, H, eps);
}

ZLLM_API int zllm_rmsnorm(const float* x, const int* rows, const void* w, void* y, int T, int H, float eps, int w_bf16, int out_bf16,
                          void* stream) {
    if (T <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (w_bf16 && out_bf16) return launch_rmsnorm<bf16, bf16>(x, rows, w, y, T, H, eps, s);
    if (w_bf16) return launch_rmsnorm<bf16, float>(x, rows, w, y, T, H, eps, s);
    if (out_bf16) return launch_rmsnorm<float, bf16>(x, rows, w, y, T, H, eps, s);
    return launch_rmsnorm<float, float>(x, rows, w, y, T, H, eps, s);
}

// ---------------------------------------------------------------- silu * up
template <typename AT>
__global__ void silu_mul_kernel(const AT* g, const AT* u, AT* o, size_t n) {
    pdl_trigger();
    pdl_wait();
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float a = to_f32(g[i]);
        o[i] = from_f32<AT>(a / (1.f + expf(-a)) * to_f32(u[i]));
    }
}

ZLLM_API int zllm_silu_mul(const void* g, const void* u, void* o, long long n, int is_bf16, void* stream) {
    if (n <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    unsigned blocks = (unsigned)((n + 255) / 256);
    if (is_bf16) return launch_pdl(silu_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (const bf16*)g, (const bf16*)u, (bf16*)o, (size_t)n);
    return launch_pdl(silu_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, (const float*)g, (const float*)u, (float*)o, (size_t)n);
}

// ---------------------------------------------------------------- gather rows (float32)
__global__ void gather_rows_kernel(const float* x, const int* rows, float* out,
                                   int H) {
    pdl_trigger();
    pdl_wait();
    const float* src = x + (size_t)rows[blockIdx.x] * H;
    float* dst = out + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
}

ZLLM_API int zllm_gather_rows(const float* x, const int* rows, float* out, int R, int H, void* stream) {
    if (R <= 0) return 0;
    return launch_pdl(gather_rows_kernel, dim3(R), dim3(256), 0, (cudaStream_t)stream, x, rows, out, H);
}

// ---------------------------------------------------------------- rotary + cache write
// qkv [T, (nq + 2 nkv) * hd]: q heads, then k heads, then v heads.  q and k are
// rotated in place over their first rot_dim entries; then (store != 0 and slot >= 0)
// k and v of the row go to the page of its position:
//   page = table[slot * max_blocks + pos / bs];  element [page][kv head][pos % bs][d].
// cos/sin: [max_pos, rot_dim/2] float32 tables of pos * theta_j (null: no rotation).
template <typename AT>
__global__ void rope_kv_store_kernel(AT* qkv, const int* positions,
                                     const int* row_slot, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, int rot_dim, int interleaved,
                                     AT* k_pages, AT* v_pages,
                                     const int* __restrict__ table, int max_blocks, int bs, int nq, int nkv, int hd,
                                     int store) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int slot = row_slot[t];
    if (slot < 0) return;                       // padding row of a graph bucket
    const int pos = positions[t];
    AT* row = qkv + (size_t)t * (nq + 2 * nkv) * hd;
    const int half = rot_dim >> 1;
    if (cos_t != nullptr) {
        const float* c = cos_t + (size_t)pos * half;
        const float* s = sin_t + (size_t)pos * half;
        const int pairs = (nq + nkv) * half;
        for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
            const int head = i / half, j = i - head * half;
            AT* h = row + (size_t)head * hd;
            const int ia = interleaved ? 2 * j : j;
            const int ib = interleaved ? 2 * j + 1 : j + half;
            const float a = to_f32(h[ia]), b = to_f32(h[ib]);
            const float cj = c[j], sj = s[j];
            h[ia] = from_f32<AT>(a * cj - b * sj);
            h[ib] = from_f32<AT>(a * sj + b * cj);
        }
    }
    if (!store) return;
    __syncthreads();                            // rotated k visible to all threads of the row
    const int page = table[(size_t)slot * max_blocks + pos / bs];
    if (page < 0) return;                       // host guarantees a page; never write through a bad id
    const int off = pos % bs;
    const AT* k = row + (size_t)nq * hd;
    const AT* v = k + (size_t)nkv * hd;
    for (int i = threadIdx.x; i < nkv * hd; i += blockDim.x) {
        const int kvh = i / hd, d = i - kvh * hd;
        const size_t dst = (((size_t)page * nkv + kvh) * bs + off) * hd + d;
        k_pages[dst] = k[i];
        v_pages[dst] = v[i];
    }
}

// bfloat16, half-split pairing over the whole head, head_dim % 16 == 0: 16-byte accesses.
// One thread rotates 8 pairs (j..j+7, j+half..j+half+7) of one head, or copies 8 values of v.
__global__ void __launch_bounds__(256) rope_kv_store_vec_kernel(bf16* qkv, const int* positions,
                                                                const int* row_slot,
                                                                const float* __restrict__ cos_t,
                                                                const float* __restrict__ sin_t,
                                                                bf16* k_pages, bf16* v_pages,
                                                                const int* __restrict__ table, int max_blocks, int bs,
                                                                int nq, int nkv, int hd, int store) {
    // The row's slot, position and page and the thread's first rotation factors are inputs of the
    // step (no kernel of the step writes them): they are fetched BEFORE the wait on the kernel
    // before, three dependent round trips that then cost nothing; after the wait only qkv is read.
    pdl_trigger();
    const int t = blockIdx.x;
    const int slot = row_slot[t];
    const int pos = positions[t];
    const int half = hd >> 1;
    const int per_head = half >> 3;                                  // 8-pair groups per rotated head
    size_t kv_base = 0;
    bool have_page = false;
    if (store && slot >= 0) {
        const int page = table[(size_t)slot * max_blocks + pos / bs];
        have_page = page >= 0;
        kv_base = ((size_t)(have_page ? page : 0) * nkv * bs + (size_t)(pos % bs)) * hd;   // + kvh * bs * hd
    }
    const int n_rot = (nq + nkv) * per_head;
    const int n_v = store ? nkv * (hd >> 3) : 0;
    auto factors = [&](int i, float (&c)[8], float (&sn)[8]) {
        if (cos_t != nullptr && i < n_rot) {
            const int head = i / per_head, j = (i - head * per_head) * 8;
            const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j);
            const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j);
            const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
            c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
            sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) { c[e] = 1.f; sn[e] = 0.f; }
        }
    };
    float c[8], sn[8];
    if (slot >= 0) factors(threadIdx.x, c, sn);
    pdl_wait();
    if (slot < 0) return;
    bf16* row = qkv + (size_t)t * (nq + 2 * nkv) * hd;
    for (int i = threadIdx.x; i < n_rot + n_v; i += blockDim.x) {
        if (i < n_rot) {
            const int head = i / per_head, j = (i - head * per_head) * 8;
            bf16* h = row + (size_t)head * hd;
            uint4 ra = *reinterpret_cast<uint4*>(h + j), rb = *reinterpret_cast<uint4*>(h + j + half);
            if (i != (int)threadIdx.x) factors(i, c, sn);
            __nv_bfloat162* pa = reinterpret_cast<__nv_bfloat162*>(&ra);
            __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&rb);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(pa[e]), b = __bfloat1622float2(pb[e]);
                pa[e] = __floats2bfloat162_rn(a.x * c[2 * e] - b.x * sn[2 * e], a.y * c[2 * e + 1] - b.y * sn[2 * e + 1]);
                pb[e] = __floats2bfloat162_rn(a.x * sn[2 * e] + b.x * c[2 * e], a.y * sn[2 * e + 1] + b.y * c[2 * e + 1]);
            }
            *reinterpret_cast<uint4*>(h + j) = ra;
            *reinterpret_cast<uint4*>(h + j + half) = rb;
            if (head >= nq && have_page) {
                bf16* dst = k_pages + kv_base + (size_t)(head - nq) * bs * hd;
                *reinterpret_cast<uint4*>(dst + j) = ra;
                *reinterpret_cast<uint4*>(dst + j + half) = rb;
            }
        } else if (have_page) {
            const int vi = i - n_rot;
            const int kvh = vi / (hd >> 3), d = (vi - kvh * (hd >> 3)) * 8;
            const uint4 v = *reinterpret_cast<const uint4*>(row + (size_t)(nq + nkv + kvh) * hd + d);
            *reinterpret_cast<uint4*>(v_pages + kv_base + (size_t)kvh * bs * hd + d) = v;
        }
    }
}

ZLLM_API int zllm_rope_kv_store(void* qkv, const int* positions, const int* row_slot, const float* cos_t,
                                const float* sin_t, int rot_dim, int interleaved, void* k_pages, void* v_pages,
                                const int* table, int max_blocks, int bs, int T, int nq, int nkv, int hd, int store,
                                int is_bf16, void* stream) {
    if (T <= 0) return 0;
    if (rot_dim > hd || (rot_dim & 1)) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    if (is_bf16 && !interleaved && hd % 16 == 0 && (cos_t == nullptr || rot_dim == hd) && ((uintptr_t)qkv % 16 == 0) &&
        (!store || (((uintptr_t)k_pages | (uintptr_t)v_pages) % 16 == 0)))
        return launch_pdl(rope_kv_store_vec_kernel, dim3(T), dim3(256), 0, s, (bf16*)qkv, positions, row_slot, cos_t,
                          sin_t, (bf16*)k_pages, (bf16*)v_pages, table, max_blocks, bs, nq, nkv, hd, store);
    if (is_bf16)
        return launch_pdl(rope_kv_store_kernel<bf16>, dim3(T), dim3(256), 0, s, (bf16*)qkv, positions, row_slot, cos_t,
                          sin_t, rot_dim, interleaved, (bf16*)k_pages, (bf16*)v_pages, table, max_blocks, bs, nq, nkv,
                          hd, store);
    return launch_pdl(rope_kv_store_kernel<float>, dim3(T), dim3(256), 0, s, (float*)qkv, positions, row_slot, cos_t,
                      sin_t, rot_dim, interleaved, (float*)k_pages, (float*)v_pages, table, max_blocks, bs, nq, nkv, hd,
                      store);
}
