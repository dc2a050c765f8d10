// The decode step's products, fused with what stands before and after them (M <= 16 rows).
//
//   out = epilogue( [rmsnorm](x) W^T )
//
// A decode step of a small model is a chain of ~10 dependent kernels per layer, each far
// too short to fill the GPU; what it costs is the length of the chain.  zllm met the same
// on its hardware and fused RoPE into the QKV matvec epilogue
// (src/backend/vulkan/shaders/decode_matvec_q4k_rope.comp:1-51), the residual add into the
// O and down products (src/backend/gpu/mod.rs:2492-2497) and SiLU-mul into the gate/up
// product (src/backend/vulkan/mod.rs:1141-1167); folding RMSNorm into a matvec's consumer
// lost there because it was recomputed per output row (BENCHMARKS.md:152-155).  Here a CTA
// owns 16 output rows and ALL of K, so it sees whole rows of x: the norm costs one pass over
// x per CTA (x is at most 16 rows), the sum of squares is taken while x is staged, and the
// scalar 1/rms is applied to the accumulators at the end.
//
// Layout of the work: one CTA = 16 weight rows; its 8 warps split K (256 k per warp per pass
// of 2048); each warp streams its weights straight from global memory into mma.sync
// fragments (because the order of k inside a tensor-core step is free as long as both operands agree,
// lane (g, t) takes the 16 consecutive k at k0 + 16 t of rows g and g + 8: no shuffles, no ldmatrix) and stages its own slice
// of x in its own shared memory, so no CTA-wide barrier is needed until the 8 partial tiles
// are summed, in warp order, through shared memory.  No cluster, no scratch, deterministic;
// a row of x never mixes with another row.
//
// Epilogues: store, add into the float32 residual, swiglu (the 16 rows are 8 gate + 8 up
// rows), and rope: the 16 rows of a tile are the 8 rotation pairs (j, j + hd/2) of one head,
// so the pair sits in one thread after the reduction; the rotated q goes to the qkv buffer,
// the rotated k and the v go straight to their cache page.
#include "common.cuh"
#include <cuda_pipeline.h>
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define MODE_STORE 0
#define MODE_ADD 1
#define MODE_SWIGLU 2
#define MODE_ROPE 3

#define GD_WARPS 8
#define GD_KW 256                       // k per warp per pass
#define GD_PASS (GD_WARPS * GD_KW)      // k per pass of the CTA
#define GD_XSTRIDE (GD_KW + 8)

struct GemmDecodeParams {
    const void* x;          // [M, K] bf16, or float32 when norm_w != nullptr
    const void* norm_w;     // [K] rmsnorm weight (nullptr: x is used as it is)
    int norm_w_bf16;
    float eps;
    const bf16* w;          // [w_rows, K]
    void* out;
    int M, N, K, mode, out_bf16, w_rows;
    // rope epilogue
    const int* positions;
    const int* row_slot;
    const float* cos_t;
    const float* sin_t;
    int interleaved, nq, nkv, hd;
    bf16* k_pages;
    bf16* v_pages;
    const int* table;
    int max_blocks, bs, store;
    int wide;               // weights may be read 32 bytes at a time
    int ksplit;             // 1, or 2: the passes over K are shared by the two CTAs of a cluster
};

__device__ __forceinline__ void gd_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 gd_ldg(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
// 32 consecutive bytes in one request (a whole sector per lane; sm_100 has 256-bit loads)
__device__ __forceinline__ void gd_ldg256(const void* p, uint4& lo, uint4& hi) {
    asm volatile("ld.global.nc.L1::no_allocate.v8.u32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];\n"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w), "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w) : "l"(p));
}
__device__ __forceinline__ unsigned gd_pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&v);
}

// Which weight rows the tile's fragment rows g and g + 8 are.  Plain: 16 consecutive rows.
// Rope: tile = (head, part); q and k heads pair row j with j + hd/2 (or 2j with 2j + 1 when
// interleaved); v heads are plain.
__device__ __forceinline__ void gd_rows(const GemmDecodeParams& p, int tile, int g, int& ra, int& rb) {
    if (p.mode != MODE_ROPE) {
        ra = tile * 16 + g;
        rb = ra + 8;
        return;
    }
    const int tiles_per_head = p.hd / 16;
    const int head = tile / tiles_per_head, part = tile - head * tiles_per_head;
    const int base = head * p.hd;
    if (head >= p.nq + p.nkv) {
        ra = base + part * 16 + g;
        rb = ra + 8;
    } else if (p.interleaved) {
        ra = base + part * 16 + 2 * g;
        rb = ra + 1;
    } else {
        ra = base + part * 8 + g;
        rb = ra + p.hd / 2;
    }
}

// NT: 8-row tiles of x (M <= 8 NT);  RT: 16-row weight tiles per CTA -- x is staged once per CTA
// and pass, so more tiles per CTA mean less traffic for x (which every CTA reads in full).
template <int NT, int RT, bool FUSE_NORM>
__global__ void __launch_bounds__(GD_WARPS * 32, 2) gemm_decode_kernel(const GemmDecodeParams p) {
    constexpr int MP = NT * 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* xs_all = reinterpret_cast<bf16*>(smem_raw);                        // [warps][MP][GD_XSTRIDE]
    float* red = reinterpret_cast<float*>(smem_raw);                         // [warps][RT * 16][MP + 1], after the loop
    __shared__ float ss_part[GD_WARPS][MP];
    __shared__ float inv_rms[MP];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    // ksplit == 2 (a matrix with few rows and a long K: too few CTAs to fill the memory system):
    // CTAs 2i and 2i + 1 form a cluster, take the even and the odd passes over K of the same rows,
    // and rank 0 adds rank 1's partial tile (through distributed shared memory, after its own, so
    // the order is fixed) before the epilogue.
    const int ksplit = p.ksplit, crank = ksplit > 1 ? (int)(blockIdx.x % ksplit) : 0;
    const int tile0 = (int)(blockIdx.x / ksplit) * RT;
    const int M = p.M, K = p.K;
    bf16* xs = xs_all + (size_t)warp * MP * GD_XSTRIDE;
    float acc[RT][NT][4];
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int i = 0; i < NT; ++i) acc[r][i][0] = acc[r][i][1] = acc[r][i][2] = acc[r][i][3] = 0.f;
    float ss[MP];                                                            // FUSE_NORM: this lane's share of sum x^2
#pragma unroll
    for (int m = 0; m < MP; ++m) ss[m] = 0.f;

    uint4 fa[4][2], fb[4][2];
    auto load_w = [&](int r, int kb) {
        int ra, rb;
        gd_rows(p, tile0 + r, g, ra, rb);
        const bool va = ra < p.w_rows, vb = rb < p.w_rows;
        const bf16* wa = p.w + (size_t)(va ? ra : 0) * K;
        const bf16* wb = p.w + (size_t)(vb ? rb : 0) * K;
        if (p.wide) {                                                        // K % 16 == 0, rows 32-byte aligned
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const int k = kb + s * 64 + t * 16;
                if (va && k < K) gd_ldg256(wa + k, fa[s][0], fa[s][1]);
                else fa[s][0] = fa[s][1] = make_uint4(0, 0, 0, 0);
                if (vb && k < K) gd_ldg256(wb + k, fb[s][0], fb[s][1]);
                else fb[s][0] = fb[s][1] = make_uint4(0, 0, 0, 0);
            }
            return;
        }
#pragma unroll
        for (int s = 0; s < 4; ++s)
#pragma unroll
            for (int hf = 0; hf < 2; ++hf) {
                const int k = kb + s * 64 + t * 16 + hf * 8;
                fa[s][hf] = (va && k < K) ? gd_ldg(wa + k) : make_uint4(0, 0, 0, 0);
                fb[s][hf] = (vb && k < K) ? gd_ldg(wb + k) : make_uint4(0, 0, 0, 0);
            }
    };
    const int n_pass = (K + GD_PASS - 1) / GD_PASS;
    // weights do not depend on the kernel before: fetch the first tile of the first pass, ask L2
    // for the rest of this CTA's weights, then wait
    pdl_trigger();
    load_w(0, crank * GD_PASS + warp * GD_KW);
    for (int r = 0; r < RT; ++r) {
        int ra, rb;
        gd_rows(p, tile0 + r, g, ra, rb);
        for (int ps = crank + (r == 0 ? ksplit : 0); ps < n_pass; ps += ksplit) {
            const int k = ps * GD_PASS + warp * GD_KW + t * 64;
            if (k < K) {
                if (ra < p.w_rows) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.w + (size_t)ra * K + k));
                if (rb < p.w_rows) asm volatile("prefetch.global.L2 [%0];" ::"l"(p.w + (size_t)rb * K + k));
            }
        }
    }
    pdl_wait();

    // What the epilogue of the CTA's first tile will need from global memory is requested now, so
    // that it is there when the products are done instead of costing the kernel's tail up to three
    // round trips one after the other (slot -> position -> page and rotation): the old residual
    // (add), or the row's slot, position, page and rotation pair (rope).  blockDim covers every
    // (row, weight row) of a tile, so a thread's place in the epilogue is known: i = threadIdx.x.
    float e_cur = 0.f, e_cos = 1.f, e_sin = 0.f;
    int e_slot = -1, e_pos = 0, e_page = -1;
    if (crank == 0 && p.mode == MODE_ADD && (int)threadIdx.x < 16 * M) {
        const int n = tile0 * 16 + (threadIdx.x & 15);
        if (n < p.N) e_cur = reinterpret_cast<const float*>(p.out)[(size_t)(threadIdx.x >> 4) * p.N + n];
    }
    if (p.mode == MODE_ROPE && (int)threadIdx.x < 8 * M) {
        const int m = threadIdx.x >> 3, j = threadIdx.x & 7;
        e_slot = p.row_slot[m];
        e_pos = p.positions[m];
        if (e_slot >= 0) {
            if (p.store) e_page = p.table[(size_t)e_slot * p.max_blocks + e_pos / p.bs];
            const int tiles_per_head = p.hd / 16;
            const int head = tile0 / tiles_per_head, part = tile0 - head * tiles_per_head;
            if (head < p.nq + p.nkv && p.cos_t != nullptr) {
                const int jj = part * 8 + j;                                 // index of the pair, in both layouts
                e_cos = p.cos_t[(size_t)e_pos * (p.hd / 2) + jj];
                e_sin = p.sin_t[(size_t)e_pos * (p.hd / 2) + jj];
            }
        }
    }

    for (int ps = crank; ps < n_pass; ps += ksplit) {
        const int kb = ps * GD_PASS + warp * GD_KW;                          // this warp's 256 k of the pass
        // stage x[0..M)[kb .. kb+256) as bf16; lane takes 8 consecutive k of every row
        const int kx = kb + lane * 8;
        if (FUSE_NORM) {
            float gw[8];
            if (kx < K) {
                if (p.norm_w_bf16) {
                    const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(p.norm_w) + kx);
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                    for (int i = 0; i < 4; ++i) { float2 f = __bfloat1622float2(h[i]); gw[2 * i] = f.x; gw[2 * i + 1] = f.y; }
                } else {
                    const float4 g0 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.norm_w) + kx);
                    const float4 g1 = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.norm_w) + kx + 4);
                    gw[0] = g0.x; gw[1] = g0.y; gw[2] = g0.z; gw[3] = g0.w; gw[4] = g1.x; gw[5] = g1.y; gw[6] = g1.z; gw[7] = g1.w;
                }
            }
#pragma unroll
            for (int m = 0; m < MP; ++m) {
                uint4 pk = make_uint4(0, 0, 0, 0);
                if (m < M && kx < K) {
                    const float* xr = reinterpret_cast<const float*>(p.x) + (size_t)m * K + kx;
                    const float4 a = *reinterpret_cast<const float4*>(xr);
                    const float4 b = *reinterpret_cast<const float4*>(xr + 4);
                    ss[m] += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w + b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
                    pk.x = gd_pack(a.x * gw[0], a.y * gw[1]);
                    pk.y = gd_pack(a.z * gw[2], a.w * gw[3]);
                    pk.z = gd_pack(b.x * gw[4], b.y * gw[5]);
                    pk.w = gd_pack(b.z * gw[6], b.w * gw[7]);
                }
                *reinterpret_cast<uint4*>(xs + (size_t)m * GD_XSTRIDE + lane * 8) = pk;
            }
        } else {
#pragma unroll
            for (int m = 0; m < MP; ++m) {
                bf16* d = xs + (size_t)m * GD_XSTRIDE + lane * 8;
                if (m < M && kx < K)
                    __pipeline_memcpy_async(d, reinterpret_cast<const bf16*>(p.x) + (size_t)m * K + kx, 16);
                else
                    *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
            }
            __pipeline_commit();
            __pipeline_wait_prior(0);
        }
        __syncwarp();
#pragma unroll
        for (int r = 0; r < RT; ++r) {
            if (r > 0 || ps > crank) load_w(r, kb);
#pragma unroll
            for (int s = 0; s < 4; ++s)
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {
                    const uint4 A = fa[s][hf], B = fb[s][hf];
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) {
                        const uint4 X = *reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + g) * GD_XSTRIDE +
                                                                        s * 64 + t * 16 + hf * 8);
                        gd_mma(acc[r][nt], A.x, B.x, A.y, B.y, X.x, X.y);
                        gd_mma(acc[r][nt], A.z, B.z, A.w, B.w, X.z, X.w);
                    }
                }
        }
        __syncwarp();                                                        // the slice is overwritten by the next pass
    }
    // ---- sum the 8 warps' partial tiles (and sums of squares) in warp order ----
    if (FUSE_NORM) {
#pragma unroll
        for (int m = 0; m < MP; ++m) {
            const float v = warp_sum(ss[m]);
            if (lane == 0) ss_part[warp][m] = v;
        }
    }
    __syncthreads();                                                         // every warp is done with its x slice
#pragma unroll
    for (int r = 0; r < RT; ++r)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int m = nt * 8 + 2 * t;
            float* r0 = red + ((size_t)warp * RT * 16 + r * 16 + g) * (MP + 1) + m;
            float* r1 = r0 + 8 * (MP + 1);
            r0[0] = acc[r][nt][0]; r0[1] = acc[r][nt][1];
            r1[0] = acc[r][nt][2]; r1[1] = acc[r][nt][3];
        }
    if (FUSE_NORM && threadIdx.x < MP) {
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < GD_WARPS; ++w) tot += ss_part[w][threadIdx.x];
        inv_rms[threadIdx.x] = rsqrtf(tot / (float)K + p.eps);
    }
    __syncthreads();
    const float* red1 = nullptr;                                             // rank 1's partial tiles, seen from rank 0
    if (ksplit > 1) {
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        red1 = cluster.map_shared_rank(red, 1);
    }
    int rt_cur = 0;                                                          // the tile the epilogue is writing
    auto total = [&](int r16, int m) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < GD_WARPS; ++w) v += red[((size_t)w * RT * 16 + rt_cur * 16 + r16) * (MP + 1) + m];
        if (red1 != nullptr) {
#pragma unroll
            for (int w = 0; w < GD_WARPS; ++w) v += red1[((size_t)w * RT * 16 + rt_cur * 16 + r16) * (MP + 1) + m];
        }
        return FUSE_NORM ? v * inv_rms[m] : v;
    };
    const int mode = p.mode;
    for (rt_cur = 0; rt_cur < RT && crank == 0; ++rt_cur) {
    const int tile = tile0 + rt_cur;
    if (tile * 16 >= p.w_rows) break;
    if (mode == MODE_STORE || mode == MODE_ADD) {
        for (int i = threadIdx.x; i < 16 * M; i += blockDim.x) {
            const int m = i >> 4, r = i & 15;
            const int n = tile * 16 + r;
            if (n >= p.N) continue;
            const float v = total(r, m);
            const size_t o = (size_t)m * p.N + n;
            if (mode == MODE_ADD) {
                // (i == threadIdx.x: one pass of this loop covers a tile)
                if (rt_cur == 0) reinterpret_cast<float*>(p.out)[o] = e_cur + v;
                else reinterpret_cast<float*>(p.out)[o] += v;
            } else if (p.out_bf16) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(p.out)[o] = v;
        }
    } else if (mode == MODE_SWIGLU) {
        for (int i = threadIdx.x; i < 8 * M; i += blockDim.x) {
            const int m = i >> 3, j = i & 7;
            const int col = tile * 8 + j;
            if (col >= p.N) continue;
            const float gt = total(j, m), up = total(j + 8, m);
            const float v = gt / (1.f + expf(-gt)) * up;
            if (p.out_bf16) reinterpret_cast<bf16*>(p.out)[(size_t)m * p.N + col] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(p.out)[(size_t)m * p.N + col] = v;
        }
    } else {   // MODE_ROPE
        const int tiles_per_head = p.hd / 16;
        const int head = tile / tiles_per_head, part = tile - head * tiles_per_head;
        const int half = p.hd / 2;
        const bool rotated = head < p.nq + p.nkv;
        for (int i = threadIdx.x; i < 8 * M; i += blockDim.x) {
            const int m = i >> 3, j = i & 7;
            const int slot = e_slot;                                         // (i == threadIdx.x)
            if (slot < 0) continue;                                          // padding row of a graph bucket
            float a = total(j, m), b = total(j + 8, m);
            int da, db;                                                      // dims within the head
            if (!rotated) { da = part * 16 + j; db = da + 8; }
            else if (p.interleaved) { da = part * 16 + 2 * j; db = da + 1; }
            else { da = part * 8 + j; db = da + half; }
            const int pos = e_pos;
            if (rotated && p.cos_t != nullptr) {
                const int jj = p.interleaved ? (da >> 1) : da;               // index of the pair
                float c = e_cos, s = e_sin;
                if (rt_cur > 0) { c = p.cos_t[(size_t)pos * half + jj]; s = p.sin_t[(size_t)pos * half + jj]; }
                const float ar = a * c - b * s, br = a * s + b * c;
                a = ar; b = br;
            }
            const bf16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
            if (head < p.nq + p.nkv) {                                       // q and k also go to the qkv buffer
                bf16* o = reinterpret_cast<bf16*>(p.out) + (size_t)m * p.N + (size_t)head * p.hd;
                o[da] = ha; o[db] = hb;
            }
            if (head >= p.nq && p.store) {
                const int page = e_page;
                if (page < 0) continue;
                const bool is_k = head < p.nq + p.nkv;
                const int kvh = is_k ? head - p.nq : head - p.nq - p.nkv;
                bf16* dst = (is_k ? p.k_pages : p.v_pages) + (((size_t)page * p.nkv + kvh) * p.bs + pos % p.bs) * p.hd;
                dst[da] = ha; dst[db] = hb;
            }
        }
    }
    }   // tiles of the CTA
    if (ksplit > 1) cg::this_cluster().sync();                               // rank 0 may still be reading rank 1's tiles
}

template <int NT, int RT, bool FUSE_NORM>
static int launch_gd(const GemmDecodeParams& p, cudaStream_t s) {
    constexpr int MP = NT * 8;
    size_t smem = (size_t)GD_WARPS * MP * GD_XSTRIDE * sizeof(bf16);
    const size_t red = (size_t)GD_WARPS * RT * 16 * (MP + 1) * sizeof(float);
    if (red > smem) smem = red;
    auto kern = gemm_decode_kernel<NT, RT, FUSE_NORM>;
    static bool attr_set = false;                                        // (smem depends on the template only)
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    const int tiles = (p.w_rows + 15) / 16;
    const int groups = (tiles + RT - 1) / RT;
    if (p.ksplit <= 1) return launch_pdl(kern, dim3(groups), dim3(GD_WARPS * 32), smem, s, p);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(groups * p.ksplit);
    cfg.blockDim = dim3(GD_WARPS * 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = p.ksplit;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, p);
}

template <int NT, bool FUSE_NORM>
static int launch_gd_rt(const GemmDecodeParams& p, cudaStream_t s) {
    // more weight rows per CTA while about two CTAs per SM remain: depends on the sizes only
    const int tiles = (p.w_rows + 15) / 16;
    if (tiles >= 4 * 256) return launch_gd<NT, 4, FUSE_NORM>(p, s);
    if (tiles >= 2 * 256) return launch_gd<NT, 2, FUSE_NORM>(p, s);
    return launch_gd<NT, 1, FUSE_NORM>(p, s);
}

// See GemmDecodeParams.  M <= 16; K % 8 == 0; 16-byte aligned operands.
// mode 3 (rope): N = (nq + 2 nkv) * hd, hd % 16 == 0, rotation over the whole head.
ZLLM_API int zllm_gemm_decode(const void* x, const void* norm_w, int norm_w_bf16, float eps, const void* w, void* out,
                              int M, int N, int K, int mode, int out_bf16, const int* positions, const int* row_slot,
                              const float* cos_t, const float* sin_t, int interleaved, int nq, int nkv, int hd,
                              void* k_pages, void* v_pages, const int* table, int max_blocks, int bs, int store,
                              void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K <= 0 || (K % 8) || mode < 0 || mode > 3) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_ADD && out_bf16) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_SWIGLU && (N % 8)) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_ROPE && (hd % 16 || N != (nq + 2 * nkv) * hd || !out_bf16)) return ZLLM_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w | (uintptr_t)norm_w) & 15) return ZLLM_ERR_UNSUPPORTED;
    GemmDecodeParams p;
    p.x = x; p.norm_w = norm_w; p.norm_w_bf16 = norm_w_bf16; p.eps = eps; p.w = (const bf16*)w; p.out = out;
    p.M = M; p.N = N; p.K = K; p.mode = mode; p.out_bf16 = out_bf16;
    p.w_rows = mode == MODE_SWIGLU ? 2 * N : N;
    p.positions = positions; p.row_slot = row_slot; p.cos_t = cos_t; p.sin_t = sin_t; p.interleaved = interleaved;
    p.nq = nq; p.nkv = nkv; p.hd = hd; p.k_pages = (bf16*)k_pages; p.v_pages = (bf16*)v_pages; p.table = table;
    p.max_blocks = max_blocks; p.bs = bs; p.store = store;
    p.wide = (K % 16 == 0) && (((uintptr_t)w & 31) == 0);
    // few rows and at least four passes over K: two CTAs per group of rows (depends on the sizes only)
    p.ksplit = (norm_w == nullptr && (p.w_rows + 15) / 16 <= 160 && K >= 4 * GD_PASS) ? 2 : 1;
    cudaStream_t s = (cudaStream_t)stream;
    const bool fuse = norm_w != nullptr;
    if (M <= 8) return fuse ? launch_gd_rt<1, true>(p, s) : launch_gd_rt<1, false>(p, s);
    return fuse ? launch_gd_rt<2, true>(p, s) : launch_gd_rt<2, false>(p, s);
}
