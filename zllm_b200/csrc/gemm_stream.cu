// bfloat16 products for FEW rows (decode steps, 1..64 rows) on the 5th-generation tensor
// cores, built around the weight stream: out[m][n] = sum_k x[m][k] w[n][k].
//
// With few rows the product is a stream of the weight matrix through the SMs; the work is to
// keep enough bytes in flight.  The operands are swapped against the many-row kernel
// (gemm_tc.cu): the WEIGHT tile [128 rows][64 k] is the M side of tcgen05.mma and the rows of
// x (padded to NP = 16, 32 or 64) are its N side, so one CTA owns 128 weight rows and the
// accumulator D[128 lanes][NP columns] sits in tensor memory.  A TMA warp feeds a ring of
// shared-memory stages (weights 16 KB + x NP x 128 bytes, 128-byte swizzle); one thread issues
// the MMAs; tcgen05.commit frees the stages.  Two CTAs fit on an SM, so one CTA's epilogue and
// ramp hide behind the other's stream.
//
// Matrices with few rows give few CTAs, so K is split over a thread-block cluster (1, 2, 4 or
// 8 CTAs): every CTA leaves its partial tile in its own shared memory and, after a cluster
// barrier, each CTA sums one share of the tile over all ranks IN RANK ORDER through
// distributed shared memory (deterministic) and applies the epilogue: store, add into the
// float32 residual, or silu(gate) * up on rows interleaved 8 gate + 8 up.
//
// Launched with programmatic dependent launch: barriers, tensor memory and the first ring
// stages of WEIGHTS are set up and requested before the wait on the kernel before; x is
// requested after it.
//
// zllm's counterpart is its family of decode matvec shaders, which likewise are written
// around the weight stream and fuse the residual add and the activation
// (src/backend/vulkan/shaders/decode_matvec_q4k.comp:1-60, src/backend/gpu/mod.rs:2492-2497).
//
// Every wait on an mbarrier is bounded; a CTA whose wait ran out records where, still walks
// through every barrier its cluster expects, frees its tensor memory and returns.
#include "common.cuh"
#include "wait_hooks.cuh"
#include <cuda.h>
#include <cooperative_groups.h>
namespace cg = cooperative_groups;

#define MODE_STORE 0
#define MODE_ADD 1
#define MODE_SWIGLU 2

#define GS_BM 128                       // weight rows per CTA
#define GS_BK 64
#define GS_W_BYTES (GS_BM * GS_BK * 2)
#define GS_MAX_STAGES 6
#define GS_PSTR (GS_BM + 4)             // floats per row of the partial tile
#define GS_WAIT_LIMIT (1u << 24)
#define GS_THREADS 192

ZLLM_WAIT_STATE(gs, GS_WAIT_LIMIT)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int where) {
    const unsigned limit = c_gs_limit;
    for (unsigned i = 0; i < limit; ++i) {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    gs_give_up(where);
    return false;
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc,
                                       unsigned accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// K-major operand tile, 128-byte swizzle: rows of 128 bytes, groups of 8 rows 1024 bytes apart
// (start address >> 4, leading offset 1, stride offset 1024 >> 4, version 1, SWIZZLE_128B).
__device__ __forceinline__ unsigned long long umma_desc(unsigned saddr) {
    unsigned long long d = 0;
    d |= (unsigned long long)((saddr >> 4) & 0x3FFF);
    d |= (unsigned long long)1 << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}

__device__ __forceinline__ unsigned pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&v);
}

__device__ __forceinline__ void tmem_ld16(unsigned taddr, unsigned* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

struct StreamParams {
    void* out;
    int M, N, K, mode, out_bf16, w_rows;
    int k_iters, iters_per_rank;        // 64-wide k steps in all, and per rank of the cluster
    int stages;
};

template <int NP>
__global__ void __launch_bounds__(GS_THREADS) gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w,
                                                                 const __grid_constant__ CUtensorMap map_x,
                                                                 const StreamParams p) {
    constexpr int X_BYTES = NP * GS_BK * 2;
    constexpr int STAGE_BYTES = GS_W_BYTES + X_BYTES;
    constexpr int TMEM_COLS = NP < 32 ? 32 : NP;
    extern __shared__ unsigned char smem_raw[];
    cg::cluster_group cluster = cg::this_cluster();
    const int crank = (int)cluster.block_rank();
    const int csize = (int)cluster.num_blocks();
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;         // swizzled tiles need 1024-byte alignment
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const int stages = p.stages;
    float* part = reinterpret_cast<float*>(base_ptr + (size_t)stages * STAGE_BYTES);     // [NP][GS_PSTR]
    unsigned char* tail = reinterpret_cast<unsigned char*>(part + NP * GS_PSTR);
    const unsigned bars = smem_u32(tail);                                // full[stages], empty[stages], acc
    const unsigned bar_acc = bars + 8 * (2 * GS_MAX_STAGES);
    volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(tail + 8 * (2 * GS_MAX_STAGES + 1));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * GS_BM;
    const int it0 = crank * p.iters_per_rank;
    const int n_it = max(0, min(p.k_iters, it0 + p.iters_per_rank) - it0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(bars + 8 * s, 1);                                  // full: one arrive (expect_tx) + bytes
            mbar_init(bars + 8 * (GS_MAX_STAGES + s), 1);                // empty: one tcgen05.commit
        }
        mbar_init(bar_acc, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {                                                     // this warp owns the tensor memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_acc = *tmem_slot;
    pdl_trigger();

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            bool ok = true;
            const int pre = c_gs_skip ? 0 : min(stages, n_it);            // (tests: no copy is issued at all)
            // the weights do not depend on the kernel before: request the first stages, then wait
            for (int i = 0; i < pre; ++i) {
                mbar_expect_tx(bars + 8 * i, STAGE_BYTES);
                tma_load_2d(base + i * STAGE_BYTES, &map_w, (it0 + i) * GS_BK, n0, bars + 8 * i);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i)
                tma_load_2d(base + i * STAGE_BYTES + GS_W_BYTES, &map_x, (it0 + i) * GS_BK, 0, bars + 8 * i);
            int g = pre;
            for (; g < n_it; ++g) {
                const int s = g % stages;
                ok = mbar_wait(bars + 8 * (GS_MAX_STAGES + s), ((g / stages) & 1) ^ 1, 0);   // stage is free
                if (!ok) break;
                const unsigned full = bars + 8 * s;
                if (c_gs_skip) continue;
                mbar_expect_tx(full, STAGE_BYTES);
                tma_load_2d(base + s * STAGE_BYTES, &map_w, (it0 + g) * GS_BK, n0, full);
                tma_load_2d(base + s * STAGE_BYTES + GS_W_BYTES, &map_x, (it0 + g) * GS_BK, 0, full);
            }
            if (!ok && !c_gs_skip)                                       // the copies already issued must land
                for (int q = max(0, g - stages); q < g; ++q) mbar_wait(bars + 8 * (q % stages), (q / stages) & 1, 1);
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N >> 3 at [17,23), M >> 4 at [24,29)
            const unsigned idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(NP >> 3) << 17) |
                                   ((unsigned)(GS_BM >> 4) << 24);
            for (int g = 0; g < n_it; ++g) {
                const int s = g % stages;
                if (!mbar_wait(bars + 8 * s, (g / stages) & 1, 2)) break;        // operands have landed
                tc_fence_after();
                const unsigned w_addr = base + s * STAGE_BYTES;
                const unsigned long long adesc = umma_desc(w_addr);
                const unsigned long long bdesc = umma_desc(w_addr + GS_W_BYTES);
#pragma unroll
                for (int k = 0; k < GS_BK / 16; ++k)                     // 32 bytes along K per step: +2 in the address field
                    tc_mma(tmem_acc, adesc + 2 * k, bdesc + 2 * k, idesc, (g > 0 || k > 0) ? 1u : 0u);
                tc_commit(bars + 8 * (GS_MAX_STAGES + s));               // stage free when these MMAs have read it
            }
            tc_commit(bar_acc);                                          // accumulator complete (or abandoned)
        }
    } else {
        // ---------------- warps 2..5: accumulator -> partial tile in shared memory ----------------
        const int q = warp & 3;
        const int r = q * 32 + lane;                                     // weight row of the tile = TMEM lane
        pdl_wait();
        const bool ok = mbar_wait(bar_acc, 0, 3);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < NP; c += 16) {
            unsigned v[16];
            if (ok && n_it > 0) {
                tmem_ld16(tmem_acc + ((unsigned)(q * 32) << 16) + c, v);
            } else {
#pragma unroll
                for (int i = 0; i < 16; ++i) v[i] = 0u;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) part[(c + i) * GS_PSTR + r] = __uint_as_float(v[i]);
        }
        tc_fence_before();
    }
    __syncthreads();
    if (csize > 1) cluster.sync();
    pdl_wait();                                                          // every thread may touch the output below

    // ---------------- sum over the ranks in rank order; epilogue ----------------
    const float* peer[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) peer[s] = (s < csize && csize > 1) ? cluster.map_shared_rank(part, s) : part;
    auto total = [&](int m, int r) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < 8; ++s)
            if (s < csize) v += peer[s][m * GS_PSTR + r];
        return v;
    };
    const int groups = 8 / csize;                                        // 16-row groups this rank finishes
    const int M = p.M;
    auto total4 = [&](int m, int r) {                                    // r % 4 == 0: four weight rows at once
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s = 0; s < 8; ++s)
            if (s < csize) {
                const float4 a = *reinterpret_cast<const float4*>(peer[s] + m * GS_PSTR + r);
                v.x += a.x; v.y += a.y; v.z += a.z; v.w += a.w;
            }
        return v;
    };
    const bool vec = (p.N % 4 == 0) && (((uintptr_t)p.out & 15) == 0);   // four outputs per thread and access
    if (p.mode == MODE_SWIGLU && vec) {
        for (int e = threadIdx.x; e < groups * 2 * M; e += GS_THREADS) {
            const int h2 = e & 1, gi = (e >> 1) % groups, m = e / (2 * groups);
            const int j = crank + gi * csize;
            const int col = (n0 + 16 * j) / 2 + 4 * h2;
            if (col >= p.N) continue;
            const float4 gt = total4(m, 16 * j + 4 * h2), up = total4(m, 16 * j + 8 + 4 * h2);
            float4 v;
            v.x = gt.x / (1.f + expf(-gt.x)) * up.x; v.y = gt.y / (1.f + expf(-gt.y)) * up.y;
            v.z = gt.z / (1.f + expf(-gt.z)) * up.z; v.w = gt.w / (1.f + expf(-gt.w)) * up.w;
            const size_t o = (size_t)m * p.N + col;
            if (p.out_bf16) *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + o) = make_uint2(pack2(v.x, v.y), pack2(v.z, v.w));
            else *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o) = v;
        }
    } else if (p.mode == MODE_SWIGLU) {
        for (int e = threadIdx.x; e < groups * 8 * M; e += GS_THREADS) {
            const int r8 = e & 7, gi = (e >> 3) % groups, m = e / (8 * groups);
            const int j = crank + gi * csize;
            const int col = (n0 + 16 * j) / 2 + r8;
            if (col >= p.N) continue;
            const float gt = total(m, 16 * j + r8), up = total(m, 16 * j + 8 + r8);
            const float v = gt / (1.f + expf(-gt)) * up;
            if (p.out_bf16) reinterpret_cast<bf16*>(p.out)[(size_t)m * p.N + col] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(p.out)[(size_t)m * p.N + col] = v;
        }
    } else if (vec) {
        for (int e = threadIdx.x; e < groups * 4 * M; e += GS_THREADS) {
            const int q4 = e & 3, gi = (e >> 2) % groups, m = e / (4 * groups);
            const int r = 16 * (crank + gi * csize) + 4 * q4;
            const int n = n0 + r;
            if (n >= p.N) continue;
            const size_t o = (size_t)m * p.N + n;
            float4 cur = make_float4(0.f, 0.f, 0.f, 0.f);    // the old residual is requested before the ranks' partials are summed
            if (p.mode == MODE_ADD) cur = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.out) + o);
            float4 v = total4(m, r);
            if (p.mode == MODE_ADD) {
                float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o);
                v.x += cur.x; v.y += cur.y; v.z += cur.z; v.w += cur.w;
                *d = v;
            } else if (p.out_bf16) {
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(p.out) + o) = make_uint2(pack2(v.x, v.y), pack2(v.z, v.w));
            } else {
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.out) + o) = v;
            }
        }
    } else {
        for (int e = threadIdx.x; e < groups * 16 * M; e += GS_THREADS) {
            const int r16 = e & 15, gi = (e >> 4) % groups, m = e / (16 * groups);
            const int r = 16 * (crank + gi * csize) + r16;
            const int n = n0 + r;
            if (n >= p.N) continue;
            const float v = total(m, r);
            const size_t o = (size_t)m * p.N + n;
            if (p.mode == MODE_ADD) reinterpret_cast<float*>(p.out)[o] += v;
            else if (p.out_bf16) reinterpret_cast<bf16*>(p.out)[o] = __float2bfloat16_rn(v);
            else reinterpret_cast<float*>(p.out)[o] = v;
        }
    }
    if (csize > 1) cluster.sync();                                       // peers may still be reading this CTA's partials
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_acc), "r"(TMEM_COLS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// [rows, K] bfloat16 row-major; box = box_rows x 64 elements, 128-byte swizzle, zero fill outside
static int make_map(CUtensorMap* map, const void* ptr, int rows, int K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ZLLM_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {GS_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ZLLM_ERR_UNSUPPORTED;
}

template <int NP>
static int launch_stream(const CUtensorMap& map_w, const CUtensorMap& map_x, const StreamParams& p0, cudaStream_t s) {
    StreamParams p = p0;
    constexpr int STAGE_BYTES = GS_W_BYTES + NP * GS_BK * 2;
    p.stages = NP <= 16 ? 5 : NP <= 32 ? 4 : 3;                          // two CTAs per SM
    const int tiles = (p.w_rows + GS_BM - 1) / GS_BM;
    // split K over a cluster while fewer than two CTAs per SM exist; depends on the sizes only
    int csize = 1;
    while (csize < 8 && tiles * csize * 2 <= 296 && p.k_iters / (csize * 2) >= 2) csize *= 2;
    p.iters_per_rank = (p.k_iters + csize - 1) / csize;
    const size_t smem = 1024 + (size_t)p.stages * STAGE_BYTES + (size_t)NP * GS_PSTR * sizeof(float) + 8 * (2 * GS_MAX_STAGES + 1) + 16;
    auto kern = gemm_stream_kernel<NP>;
    static bool attr_set = false;                                        // (smem depends on the template only)
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(csize, tiles, 1);
    cfg.blockDim = dim3(GS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kern, map_w, map_x, p);
}

// x [M,K] bf16, w [N,K] bf16 ([2N,K] for swiglu), out [M,N] bf16 or float32.  M <= 64, K % 8 == 0,
// operands 16-byte aligned.
ZLLM_API int zllm_gemm_stream_bf16(const void* x, const void* w, void* out, int M, int N, int K, int mode, int out_bf16,
                                   void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K % 8) || mode < 0 || mode > 2) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_ADD && out_bf16) return ZLLM_ERR_UNSUPPORTED;
    if (mode == MODE_SWIGLU && (N % 8)) return ZLLM_ERR_UNSUPPORTED;
    if (((uintptr_t)x | (uintptr_t)w) & 15) return ZLLM_ERR_UNSUPPORTED;
    StreamParams p;
    p.out = out; p.M = M; p.N = N; p.K = K; p.mode = mode; p.out_bf16 = out_bf16;
    p.w_rows = mode == MODE_SWIGLU ? 2 * N : N;
    p.k_iters = (K + GS_BK - 1) / GS_BK;
    p.iters_per_rank = p.k_iters;
    p.stages = 0;
    const int NP = M <= 16 ? 16 : M <= 32 ? 32 : 64;
    CUtensorMap map_w, map_x;
    int e = make_map(&map_w, w, p.w_rows, K, GS_BM);
    if (e) return e;
    e = make_map(&map_x, x, M, K, NP);
    if (e) return e;
    cudaStream_t s = (cudaStream_t)stream;
    if (NP == 16) return launch_stream<16>(map_w, map_x, p, s);
    if (NP == 32) return launch_stream<32>(map_w, map_x, p, s);
    return launch_stream<64>(map_w, map_x, p, s);
}

ZLLM_WAIT_EXPORTS(gs, gemm_stream)
