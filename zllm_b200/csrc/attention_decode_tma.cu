// Decode attention over the paged cache with keys and values brought in by TMA.
//
// Same scheme as the decode kernel of attention_bf16.cu -- one CTA per (decoded row, kv head,
// split of 256 keys), each of the 4 warps takes 64 keys, the warps' partials are merged in warp
// order, a second kernel merges the splits -- but built for the memory system:
//  * a page of the cache, [positions][head_dim] of one kv head, is a box of a 2-D tensor map
//    over the pool, so ONE cp.async.bulk.tensor instruction brings a whole page (2 KB at 16
//    positions x 64 dims) into shared memory, 128-byte swizzled; a warp issues its 4 + 4 boxes
//    from 8 lanes and waits on its own two mbarriers (keys, values).  No per-row address
//    arithmetic, no LSU traffic for the copies;
//  * the tensor-core tiles are turned: KEYS are the 16 rows of mma.m16n8k16 and the query
//    heads of the group its 8 columns (S^T = K Q^T, O^T = V^T P^T), so a group of 4 or 8 heads
//    wastes nothing on padding rows: half the MMAs and exponentials of the other orientation.
//    P^T is moved between the two products with movmatrix (an 8 x 8 transpose in registers).
// All pages of the split are requested BEFORE the wait on the kernel before (programmatic
// dependent launch); the row's own key and value, which that kernel writes, are read with plain
// loads after the wait and stored over their stale copies in the tiles.
//
// Takes head sizes 64 and 128, groups nq/nkv <= 8, page sizes 8..256 that are powers of two,
// no window; the caller sends everything else to the kernel of attention_bf16.cu.  The cache
// pool must hold finite numbers everywhere (it is created zeroed): positions of a page beyond
// the row's own are loaded with their page and meet probability zero.
//
// zllm's counterpart: its flash-decode pair (src/backend/vulkan/shaders/
// sdpa_flash_partial2.comp:1-56, sdpa_flash_combine_h.comp:1-41).
//
// Waits on mbarriers are bounded; a wait that runs out sets a flag the host reads.
#include "attention_common.cuh"
#include "wait_hooks.cuh"
#include <cuda.h>
#include <string.h>

#define DT_WAIT_LIMIT (1u << 22)

ZLLM_WAIT_STATE(dt, DT_WAIT_LIMIT)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int where) {
    const unsigned limit = c_dt_limit;
    for (unsigned i = 0; i < limit; ++i) {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    dt_give_up(where);
    return false;
}
__device__ __forceinline__ void tma_load_2d(unsigned dst, const CUtensorMap* map, int x, int y, unsigned bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ unsigned movmatrix_trans(unsigned a) {
    unsigned d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

// BIG changes no instruction: the two instantiations only carry different preferences for the
// split of an SM's memory between L1 and shared memory (see launch_decode_tma).
// DIRECT: the grid has ONE split per row (contexts up to 256), so the CTA's merged result is the
// row's output: it is written as it is and no second kernel runs.
template <int HD, bool BIG, bool DIRECT>
__global__ void __launch_bounds__(DEC_WARPS * 32) decode_tma_kernel(
    const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
    const bf16* qkv, const int* rows, const int* positions,
    const int* row_slot, const bf16* k_pages, const bf16* v_pages,
    const int* __restrict__ table, int max_blocks, int bs, int bs_shift,
    int box_rows, int nq, int nkv, float scale, float* part_o, float* part_ml,
    int max_splits, bf16* out) {
    constexpr int NB = HD <= 64 ? 64 : 32;                   // keys per warp iteration
    constexpr int NIT = (SPLIT_KEYS / DEC_WARPS) / NB;       // iterations per warp
    constexpr int HALVES = HD / 64;                          // 128-byte column boxes per row
    constexpr int HALF_BYTES = NB * 128;                     // [NB keys][64 dims], swizzled
    constexpr int TILE_BYTES = HALVES * HALF_BYTES;          // the K (or V) tile of one warp
    constexpr int KS = HD / 16;                              // tensor-core steps along the head
    constexpr int CH = HD / 8;                               // 16-byte chunks of a row
    extern __shared__ unsigned char smem_raw[];
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const unsigned k_tile = base + warp * 2 * TILE_BYTES, v_tile = k_tile + TILE_BYTES;
    unsigned char* v_ptr = base_ptr + (size_t)warp * 2 * TILE_BYTES + TILE_BYTES;
    const unsigned bars = base + DEC_WARPS * 2 * TILE_BYTES;
    const unsigned bar_k = bars + 16 * warp, bar_v = bar_k + 8;

    pdl_trigger();
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (lane == 0) {
        mbar_init(bar_k, 1);
        mbar_init(bar_v, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const int row = rows[blockIdx.x];
    const int slot = row_slot[row];
    const int kvh = blockIdx.y, split = blockIdx.z;
    if (slot < 0) {                                          // padding row of a graph bucket
        if (DIRECT) {
            const int Gp = nq / nkv;
            for (int i = threadIdx.x; i < Gp * HD; i += blockDim.x)
                out[((size_t)row * nq + kvh * Gp) * HD + i] = __float2bfloat16_rn(0.f);
        }
        return;
    }
    const int pos = positions[row];
    const int k_first = split * SPLIT_KEYS;
    if (k_first > pos) return;                               // this split holds no key of the row
    const int G = nq / nkv;
    const int* trow = table + (size_t)slot * max_blocks;
    const int w_first = k_first + warp * (SPLIT_KEYS / DEC_WARPS);
    const bool active = w_first <= pos;                      // warp-uniform
    __syncwarp();

    // One iteration's boxes: lanes 0..15 the keys', 16..31 the values'; box = (page part, column half).
    const int n_box = (NB / box_rows) * HALVES;
    const int bidx = lane & 15, is_v = lane >> 4;
    const int pb = bidx / HALVES, half = bidx - pb * HALVES;
    const unsigned box_bytes = (unsigned)box_rows * 128u;
    // request iteration ``it``: every box that holds a key <= pos.  The box that holds pos itself is
    // requested like the others although the kernel before may still be writing that one row:
    // the row is put in place from registers after the wait (see own_row below)
    auto issue = [&](int it) {
        if (c_dt_skip) return;                               // (tests: no copy is ever in flight)
        const int key0 = w_first + it * NB;
        const int key_b0 = key0 + pb * box_rows;
        bool valid = bidx < n_box && key_b0 <= pos;
        int y = 0;
        if (valid) {
            const int page = trow[key_b0 >> bs_shift];
            valid = page >= 0;
            y = (page * nkv + kvh) * bs + (key_b0 & (bs - 1));
        }
        const unsigned m = __ballot_sync(0xffffffffu, valid);
        if (lane == 0) mbar_expect_tx(bar_k, (unsigned)__popc(m & 0xffffu) * box_bytes);
        if (lane == 16) mbar_expect_tx(bar_v, (unsigned)__popc(m >> 16) * box_bytes);
        __syncwarp();
        // boxes of V that are not loaded must not hold garbage: probability 0 x NaN is NaN
        for (int b = 0; b < n_box; ++b) {
            if ((m >> (16 + b)) & 1u) continue;
            const int pbb = b / HALVES, hb = b - pbb * HALVES;
            uint4* z = reinterpret_cast<uint4*>(v_ptr + hb * HALF_BYTES + pbb * box_rows * 128);
            for (int i = lane; i < box_rows * 8; i += 32) z[i] = make_uint4(0, 0, 0, 0);
        }
        if (valid) {
            const unsigned dst = (is_v ? v_tile : k_tile) + half * HALF_BYTES + pb * box_rows * 128;
            tma_load_2d(dst, is_v ? &map_v : &map_k, half * 64, y, is_v ? bar_v : bar_k);
        }
    };
    if (active) issue(0);
    pdl_wait();

    // query fragments (B operand): head g of the group, dims 16 ks + 2t, +1 and + 8
    unsigned qf[KS][2];
    {
        const bf16* qrow = qkv + (size_t)row * (nq + 2 * nkv) * HD + ((size_t)kvh * G + g) * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            qf[ks][0] = g < G ? *reinterpret_cast<const unsigned*>(qrow + 16 * ks + 2 * t) : 0u;
            qf[ks][1] = g < G ? *reinterpret_cast<const unsigned*>(qrow + 16 * ks + 8 + 2 * t) : 0u;
        }
    }
    // running softmax state of heads 2t and 2t + 1: max (uniform over g), this lane's share of the
    // sum, and O^T: o[dt][0..1] = (dim 16 dt + g; heads 2t, 2t + 1), o[dt][2..3] = (dim 16 dt + 8 + g; ..)
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    float o[KS][4];
#pragma unroll
    for (int i = 0; i < KS; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    const int lrow = lane & 7, lmat = lane >> 3;

#pragma unroll 1
    for (int it = 0; it < NIT && active; ++it) {
        const int key0 = w_first + it * NB;
        if (key0 > pos) break;                               // warp-uniform
        if (it > 0) {
            // the tiles are reused: the reads of the last iteration come before the new copies
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            issue(it);
        }
        // the row's own key and value (written by the kernel before this one) come by plain loads:
        // 16-byte chunk ``own_c`` of K (lanes 0 .. CH-1) or V (lanes CH .. 2 CH-1), stored over the
        // stale copy in the tile once the tile has landed
        const bool own_here = pos < key0 + NB;
        uint4 own = make_uint4(0, 0, 0, 0);
        const int own_c = lane % CH, own_v = lane / CH;
        if (own_here && lane < 2 * CH) {
            const int page = trow[pos >> bs_shift];
            if (page >= 0) {
                const size_t r = (size_t)(page * nkv + kvh) * bs + (pos & (bs - 1));
                own = __ldcg(reinterpret_cast<const uint4*>((own_v ? v_pages : k_pages) + r * HD + own_c * 8));
            }
        }
        const unsigned own_off = (unsigned)((own_c >> 3) * HALF_BYTES + (pos - key0) * 128 + (((own_c & 7) ^ ((pos - key0) & 7)) << 4));
        const unsigned parity = it & 1;
        mbar_wait(bar_k, parity, 0);
        if (own_here) {
            if (lane < CH) *reinterpret_cast<uint4*>(base_ptr + (k_tile - base) + own_off) = own;
            __syncwarp();
        }
        // S^T = K Q^T: sc[mt][0..1] = (key 16 mt + g; heads 2t, 2t + 1), sc[mt][2..3] = (key 16 mt + 8 + g; ..)
        float sc[NB / 16][4];
#pragma unroll
        for (int mt = 0; mt < NB / 16; ++mt) {
            sc[mt][0] = sc[mt][1] = sc[mt][2] = sc[mt][3] = 0.f;
            const int key = 16 * mt + (lmat & 1) * 8 + lrow;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const int chunk = 2 * ks + (lmat >> 1);      // 16-byte chunk of the row
                unsigned a[4];
                const unsigned addr = k_tile + (chunk >> 3) * HALF_BYTES + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
                mma16816(sc[mt], a, qf[ks][0], qf[ks][1]);
            }
        }
        // masking (only the block that holds pos), running max over the keys of each head
        float mx[2] = {-INFINITY, -INFINITY};
        const bool masked = key0 + NB - 1 > pos;
#pragma unroll
        for (int mt = 0; mt < NB / 16; ++mt) {
            if (masked) {
                if (key0 + 16 * mt + g > pos) sc[mt][0] = sc[mt][1] = -INFINITY;
                if (key0 + 16 * mt + 8 + g > pos) sc[mt][2] = sc[mt][3] = -INFINITY;
            }
            mx[0] = fmaxf(mx[0], fmaxf(sc[mt][0], sc[mt][2]));
            mx[1] = fmaxf(mx[1], fmaxf(sc[mt][1], sc[mt][3]));
        }
        float corr[2], msafe[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 4));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 8));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 16));
            const float m_new = fmaxf(m_run[h], mx[h] * scale);
            corr[h] = (m_new == -INFINITY) ? 1.f : ex2_approx(m_run[h] - m_new);
            msafe[h] = (m_new == -INFINITY) ? 0.f : m_new;
            m_run[h] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        unsigned pb_frag[NB / 16][2];                        // P^T as B fragments: (keys 2t, 2t+1 (+8); head g)
#pragma unroll
        for (int mt = 0; mt < NB / 16; ++mt) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float p = ex2_approx(fmaf(sc[mt][e], scale, -msafe[e & 1]));     // 2^(-inf) = 0 for hidden keys
                sc[mt][e] = p;
                rs[e & 1] += p;
            }
            pb_frag[mt][0] = movmatrix_trans(pack_bf16(sc[mt][0], sc[mt][1]));
            pb_frag[mt][1] = movmatrix_trans(pack_bf16(sc[mt][2], sc[mt][3]));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * corr[h] + rs[h];
#pragma unroll
        for (int i = 0; i < KS; ++i) {
            o[i][0] *= corr[0]; o[i][1] *= corr[1];
            o[i][2] *= corr[0]; o[i][3] *= corr[1];
        }
        mbar_wait(bar_v, parity, 1);
        if (own_here) {
            if (lane >= CH && lane < 2 * CH) *reinterpret_cast<uint4*>(base_ptr + (v_tile - base) + own_off) = own;
            __syncwarp();
        }
        // O^T += V^T P^T: A fragments of V^T by transposed ldmatrix
#pragma unroll
        for (int mt = 0; mt < NB / 16; ++mt) {
            const int key = 16 * mt + (lmat >> 1) * 8 + lrow;
#pragma unroll
            for (int dt = 0; dt < KS; ++dt) {
                const int chunk = 2 * dt + (lmat & 1);
                unsigned a[4];
                const unsigned addr = v_tile + (chunk >> 3) * HALF_BYTES + key * 128 + (((chunk & 7) ^ (key & 7)) << 4);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
                mma16816(o[dt], a, pb_frag[mt][0], pb_frag[mt][1]);
            }
        }
    }
    // this lane's share of the sums -> the heads' sums
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 4);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 8);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 16);
    }
    // merge the warps' partials in warp order
    __syncthreads();                                         // all warps are done with their tiles
    float* wm = reinterpret_cast<float*>(base_ptr);          // [warps][8]
    float* wl = wm + DEC_WARPS * 8;                          // [warps][8]
    float* wo = wl + DEC_WARPS * 8;                          // [warps][8][HD]
    if (g == 0) {
        wm[warp * 8 + 2 * t] = m_run[0]; wm[warp * 8 + 2 * t + 1] = m_run[1];
        wl[warp * 8 + 2 * t] = l_run[0]; wl[warp * 8 + 2 * t + 1] = l_run[1];
    }
#pragma unroll
    for (int dt = 0; dt < KS; ++dt) {
        float* o0 = wo + ((size_t)warp * 8 + 2 * t) * HD + 16 * dt + g;
        float* o1 = o0 + HD;
        o0[0] = o[dt][0]; o1[0] = o[dt][1];
        o0[8] = o[dt][2]; o1[8] = o[dt][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * HD; i += blockDim.x) {
        const int h = i / HD, d = i - h * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w * 8 + h]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = wm[w * 8 + h];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            L += wl[w * 8 + h] * f;
            O += wo[((size_t)w * 8 + h) * HD + d] * f;
        }
        if (DIRECT) {
            out[((size_t)row * nq + kvh * G + h) * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else {
            const size_t pi = ((size_t)blockIdx.x * nq + kvh * G + h) * max_splits + split;
            part_o[pi * HD + d] = O;
            if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
        }
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

static int box_rows_for(int bs, int hd) {
    const int nb = hd <= 64 ? 64 : 32;
    return bs < nb ? bs : nb;
}

// Writes the 128-byte tensor map of one pool of pages [num_pages][nkv][bs][hd] (bfloat16) to
// ``out_map``: a 2-D tensor of num_pages * nkv * bs rows of hd elements, boxes of
// min(bs, keys per warp iteration) rows x 64 elements, 128-byte swizzle.
ZLLM_API int zllm_attention_kv_map(void* out_map, const void* pages, long long num_pages, int nkv, int bs, int hd) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || (hd != 64 && hd != 128) || bs < 8 || bs > 256 || (bs & (bs - 1)) || ((uintptr_t)pages & 15))
        return ZLLM_ERR_UNSUPPORTED;
    alignas(64) CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)(num_pages * nkv * bs)};
    cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows_for(bs, hd)};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ZLLM_ERR_UNSUPPORTED;
    memcpy(out_map, &map, sizeof(map));
    return 0;
}

// The shared-memory carveout of this kernel decides how well the decode chain overlaps
// (measured, 1B shape): left to the driver it gets the largest carveout (3 CTAs of 66 KB), and a
// batch-8 step at context 128 takes 931 us instead of 832 us with a 60 % preference, because the
// small kernels before and after it, which run on the same SMs at the same time, then wait for
// the SM's memory to be re-split.  With thousands of CTAs the third CTA per SM is worth more than
// that (batch 64, context 4096: 2.71 ms against 3.02 ms).  So: the largest carveout when the grid
// is large or the batch is one whose products already use the large-shared-memory streaming
// kernel; 60 % otherwise.  The choice depends on the grid's size only and changes no result.
template <int HD, bool BIG, bool DIRECT>
static int launch_decode_tma_v(const CUtensorMap& mk, const CUtensorMap& mv, const void* k_pages, const void* v_pages,
                             const void* qkv, void* out, const int* rows,
                             int n_rows, const int* positions, const int* row_slot, const int* table, int max_blocks,
                             int bs, int nq, int nkv, float scale, float* part_o, float* part_ml, int n_splits,
                             int max_splits, cudaStream_t s) {
    constexpr int NB = HD <= 64 ? 64 : 32;
    const size_t smem = 1024 + (size_t)DEC_WARPS * 2 * (HD / 64) * NB * 128 + 16 * DEC_WARPS;
    auto kern = decode_tma_kernel<HD, BIG, DIRECT>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                                 BIG ? (int)cudaSharedmemCarveoutMaxShared : 60);
        if (e != cudaSuccess) return (int)e;
        attr_set = true;
    }
    dim3 grid(n_rows, nkv, n_splits);
    int rc = launch_pdl(kern, grid, dim3(DEC_WARPS * 32), smem, s, mk, mv, (const bf16*)qkv, rows, positions, row_slot,
                        (const bf16*)k_pages, (const bf16*)v_pages, table, max_blocks, bs, (int)__builtin_ctz(bs), box_rows_for(bs, HD), nq, nkv,
                        scale * 1.4426950408889634f, part_o, part_ml, max_splits, (bf16*)out);
    if (rc || DIRECT) return rc;
    return launch_combine<HD>(n_rows, nq, n_splits, s, rows, positions, row_slot, (const float*)part_o, (const float*)part_ml,
                              (bf16*)out, 0, max_splits);
}

template <int HD>
static int launch_decode_tma(const CUtensorMap& mk, const CUtensorMap& mv, const void* k_pages, const void* v_pages,
                             const void* qkv, void* out, const int* rows, int n_rows, const int* positions,
                             const int* row_slot, const int* table, int max_blocks, int bs, int nq, int nkv, float scale,
                             float* part_o, float* part_ml, int n_splits, int max_splits, cudaStream_t s) {
    const bool big = n_rows > 16 || (long long)n_rows * nkv * n_splits >= 2048;
#define DT_LAUNCH(B, D) launch_decode_tma_v<HD, B, D>(mk, mv, k_pages, v_pages, qkv, out, rows, n_rows, positions, row_slot, \
                                                      table, max_blocks, bs, nq, nkv, scale, part_o, part_ml, n_splits,     \
                                                      max_splits, s)
    if (n_splits == 1) return big ? DT_LAUNCH(true, true) : DT_LAUNCH(false, true);
    return big ? DT_LAUNCH(true, false) : DT_LAUNCH(false, false);
#undef DT_LAUNCH
}

// As zllm_attention_decode_bf16 (attention_bf16.cu) with the pools given by their tensor maps
// (zllm_attention_kv_map) beside their addresses.  hd 64 or 128, nq / nkv <= 8, bs a power of two in 8..256, no window.
ZLLM_API int zllm_attention_decode_tma(const void* qkv, void* out, const int* rows, int n_rows, const int* positions,
                                       const int* row_slot, const void* map_k, const void* map_v, const void* k_pages,
                                       const void* v_pages, const int* table,
                                       int max_blocks, int bs, int nq, int nkv, int hd, float scale, float* part_o,
                                       float* part_ml, int n_splits, int max_splits, void* stream) {
    if (n_rows <= 0) return 0;
    if (nkv <= 0 || nq % nkv || nq / nkv > 8 || n_splits <= 0 || n_splits > max_splits || n_splits > 65535 ||
        nkv > 65535 || bs < 8 || bs > 256 || (bs & (bs - 1)) || !map_k || !map_v)
        return ZLLM_ERR_UNSUPPORTED;
    alignas(64) CUtensorMap mk, mv;
    memcpy(&mk, map_k, sizeof(mk));
    memcpy(&mv, map_v, sizeof(mv));
    cudaStream_t s = (cudaStream_t)stream;
    if (hd == 64)
        return launch_decode_tma<64>(mk, mv, k_pages, v_pages, qkv, out, rows, n_rows, positions, row_slot, table, max_blocks, bs, nq, nkv,
                                     scale, part_o, part_ml, n_splits, max_splits, s);
    if (hd == 128)
        return launch_decode_tma<128>(mk, mv, k_pages, v_pages, qkv, out, rows, n_rows, positions, row_slot, table, max_blocks, bs, nq, nkv,
                                      scale, part_o, part_ml, n_splits, max_splits, s);
    return ZLLM_ERR_UNSUPPORTED;
}

ZLLM_WAIT_EXPORTS(dt, attention_decode_tma)
