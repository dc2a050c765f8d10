// bfloat16 attention over the paged cache on tensor cores (mma.sync m16n8k16), float32
// softmax and accumulation.
//
// Two kernels with one inner loop:
//  * decode: one CTA per (decoded row, kv head, split of 256 keys).  The query heads that
//    share the kv head are the 16 rows of the tensor-core tile, so keys and values are read
//    once for the whole group; each of the 4 warps takes 64 keys of the split; the warps'
//    partial (max, sum, accumulator) are merged in warp order and written as the split's
//    partial; a second kernel merges the splits in split order.  This is zllm's
//    flash-decode scheme (partial + log-sum-exp combine, src/backend/vulkan/shaders/
//    sdpa_flash_partial2.comp:1-56, sdpa_flash_combine_h.comp:1-41) on the math of its paged
//    kernel (src/backend/gpu/shaders.rs:670-725).  The split size is fixed, so how a row is
//    split depends on its own position only, never on the batch.
//  * prefill: one CTA per (tile of 128 query rows of a portion, query head); K/V tiles of 64
//    keys are gathered through the block table into a 3-stage ring in shared memory and
//    shared by the CTA's warps (two 16-row tiles each for head sizes up to 64); a portion that starts at position p
//    attends the whole prefix 0..p-1 from the cache plus its own rows causally (zllm's
//    coopmat_flash_attn.comp with its query offset, src/backend/vulkan/mod.rs:1758-1777).
//
// Scratch: the decode kernel's per-split partials live in global memory given by the
// caller: part_o [rows][nq][max_splits][hd] and part_ml [rows][nq][max_splits][2] float32.
#include "attention_common.cuh"
#include <cuda_pipeline.h>

// Running softmax state of one warp's 16-row tile: rows g and g + 8 of the lane.
template <int HD>
struct TileState {
    float m[2], l[2];
    float o[HD / 8][4];
    __device__ __forceinline__ void init() {
        m[0] = m[1] = -INFINITY;
        l[0] = l[1] = 0.f;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    }
};

// Gather NKEYS rows of K or V (keys key0 .. key0+NKEYS-1 of one request and kv head) into a
// shared tile [NKEYS][HD + 8] with 16-byte async copies by NTHREADS threads.  Keys outside
// [0, n_keys) or without a page are zero-filled.  Each thread looks up the page of its row
// once; bs_shift >= 0 when the page size is a power of two (no division).
template <int HD, int NKEYS, int NTHREADS>
__device__ __forceinline__ void gather_tile(bf16* __restrict__ tile, const bf16* __restrict__ pages,
                                            const int* __restrict__ trow, int key0, int n_keys, int bs, int bs_shift,
                                            int nkv, int kvh, int tid) {
    constexpr int CH = HD / 8;                       // 16-byte chunks per row
    constexpr int TPR = NTHREADS >= NKEYS ? NTHREADS / NKEYS : 1;     // threads per row
    constexpr int ROWS_PER_PASS = NTHREADS / TPR;
    const int part = tid % TPR;
#pragma unroll
    for (int r = tid / TPR; r < NKEYS; r += ROWS_PER_PASS) {
        const int key = key0 + r;
        bf16* dst = tile + (size_t)r * (HD + 8);
        const bf16* src = nullptr;
        if (key >= 0 && key < n_keys) {
            const int blk = bs_shift >= 0 ? (key >> bs_shift) : key / bs;
            const int off = bs_shift >= 0 ? (key & (bs - 1)) : key - blk * bs;
            const int page = trow[blk];
            if (page >= 0) src = pages + (((size_t)page * nkv + kvh) * bs + off) * HD;
        }
        if (src != nullptr) {
#pragma unroll
            for (int c = part; c < CH; c += TPR) __pipeline_memcpy_async(dst + c * 8, src + c * 8, 16);
        } else {
#pragma unroll
            for (int c = part; c < CH; c += TPR) *reinterpret_cast<uint4*>(dst + c * 8) = make_uint4(0, 0, 0, 0);
        }
    }
}

// After the scores: masking, running softmax in float32, and O += P V with V from a shared tile.
//   s       : raw scores q.k of the warp's 16 rows against the block's NB keys (C fragments)
//   vs      : shared tile [NB][HD + 8] of the block's values
//   key0    : absolute index of the block's first key
//   lo_r/hi_r : per row (index 0: row g, 1: row g + 8) the visible key range [lo, hi]
template <int HD, int NB, bool MASKED, bool WAIT_V = false>
__device__ __forceinline__ void softmax_pv(float (&s)[NB / 8][4], const bf16* __restrict__ vs, int key0,
                                           const int (&lo_r)[2], const int (&hi_r)[2], float scale,
                                           TileState<HD>& st, int lane) {
    constexpr int STR = HD + 8;
    const int t = lane & 3;
    const int lrow = lane & 7, lmat = lane >> 3;
    // running max in the scaled log2 domain (scale > 0 holds log2(e): max commutes with it);
    // only blocks that touch a row's edge of visibility pay for the masking
    float mx[2] = {-INFINITY, -INFINITY};
    if (MASKED) {
#pragma unroll
        for (int j = 0; j < NB / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const int key = key0 + 8 * j + 2 * t + (e & 1);
                if (!(key >= lo_r[r] && key <= hi_r[r])) s[j][e] = -INFINITY;
                mx[r] = fmaxf(mx[r], s[j][e]);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < NB / 8; ++j) {
            mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
            mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
        }
    }
    float corr[2], msafe[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(st.m[r], mx[r] * scale);
        corr[r] = (m_new == -INFINITY) ? 1.f : ex2_approx(st.m[r] - m_new);
        msafe[r] = (m_new == -INFINITY) ? 0.f : m_new;
        st.m[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
#pragma unroll
    for (int j = 0; j < NB / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int r = e >> 1;
            const float p = ex2_approx(fmaf(s[j][e], scale, -msafe[r]));     // 2^(-inf) = 0 for hidden keys
            s[j][e] = p;
            rs[r] += p;
        }
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
        st.l[r] = st.l[r] * corr[r] + rs[r];
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        st.o[i][0] *= corr[0]; st.o[i][1] *= corr[0];
        st.o[i][2] *= corr[1]; st.o[i][3] *= corr[1];
    }
    if (WAIT_V) {                        // the warp's own async copies of V must have landed
        __pipeline_wait_prior(0);
        __syncwarp();
    }
    // O += P V: A fragments from the probabilities, B fragments of V by transposed ldmatrix
#pragma unroll
    for (int kk = 0; kk < NB / 16; ++kk) {
        unsigned pa[4];
        pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int i = 0; i < HD / 8; i += 2) {
            // matrices: (keys 16kk.., dims 8i..), (keys 16kk+8.., dims 8i..), (keys 16kk.., dims 8i+8..), (.., +8)
            unsigned b[4];
            const bf16* p = vs + (size_t)(16 * kk + (lmat & 1) * 8 + lrow) * STR + 8 * i + (lmat >> 1) * 8;
            ldmatrix_x4_trans(b, p);
            mma16816(st.o[i], pa, b[0], b[1]);
            mma16816(st.o[i + 1], pa, b[2], b[3]);
        }
    }
}

// One block of NB keys (NB multiple of 16) against MT 16-row tiles of the warp (prefill).  The
// fragments of K and V are read from shared memory ONCE and used for all MT tiles: with MT = 2
// the shared-memory traffic per tensor-core step halves.
//   qf      : A fragments of the MT 16 x HD query tiles
//   ks, vs  : shared tiles [NB][HD + 8] of the block's keys / values
//   key0    : absolute index of the block's first key
//   lo_r/hi_r : per tile and row (index 0: row g, 1: row g + 8) the visible key range [lo, hi]
template <int HD, int NB, bool MASKED, int MT>
__device__ __forceinline__ void attend_block(const unsigned (&qf)[MT][HD / 16][4], const bf16* __restrict__ ks,
                                             const bf16* __restrict__ vs, int key0, const int (&lo_r)[MT][2],
                                             const int (&hi_r)[MT][2], float scale, TileState<HD> (&st)[MT], int lane) {
    constexpr int STR = HD + 8;
    const int t = lane & 3;
    const int lrow = lane & 7, lmat = lane >> 3;
    float s[MT][NB / 8][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int j = 0; j < NB / 8; ++j) s[mt][j][0] = s[mt][j][1] = s[mt][j][2] = s[mt][j][3] = 0.f;
    // S = Q K^T: B fragments of K by ldmatrix (rows = keys, 8 x 8 tiles along dims)
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int j = 0; j < NB / 8; j += 2) {
            // matrices: (keys 8j.., dims 16kk..), (keys 8j.., dims 16kk+8..), (keys 8j+8.., dims 16kk..), (.., +8)
            unsigned b[4];
            const bf16* p = ks + (size_t)(8 * j + (lmat >> 1) * 8 + lrow) * STR + 16 * kk + (lmat & 1) * 8;
            ldmatrix_x4(b, p);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma16816(s[mt][j], qf[mt][kk], b[0], b[1]);
                mma16816(s[mt][j + 1], qf[mt][kk], b[2], b[3]);
            }
        }
    }
    // masking and running softmax per tile, in the scaled log2 domain
    unsigned pa[MT][NB / 16][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        float mx[2] = {-INFINITY, -INFINITY};
        if (MASKED) {
#pragma unroll
            for (int j = 0; j < NB / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    const int key = key0 + 8 * j + 2 * t + (e & 1);
                    if (!(key >= lo_r[mt][r] && key <= hi_r[mt][r])) s[mt][j][e] = -INFINITY;
                    mx[r] = fmaxf(mx[r], s[mt][j][e]);
                }
        } else {
#pragma unroll
            for (int j = 0; j < NB / 8; ++j) {
                mx[0] = fmaxf(mx[0], fmaxf(s[mt][j][0], s[mt][j][1]));
                mx[1] = fmaxf(mx[1], fmaxf(s[mt][j][2], s[mt][j][3]));
            }
        }
        float corr[2], msafe[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(st[mt].m[r], mx[r] * scale);
            corr[r] = (m_new == -INFINITY) ? 1.f : ex2_approx(st[mt].m[r] - m_new);
            msafe[r] = (m_new == -INFINITY) ? 0.f : m_new;
            st[mt].m[r] = m_new;
        }
        float rs[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < NB / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const float pr = ex2_approx(fmaf(s[mt][j][e], scale, -msafe[r]));     // 2^(-inf) = 0 for hidden keys
                s[mt][j][e] = pr;
                rs[r] += pr;
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            st[mt].l[r] = st[mt].l[r] * corr[r] + rs[r];
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            st[mt].o[i][0] *= corr[0]; st[mt].o[i][1] *= corr[0];
            st[mt].o[i][2] *= corr[1]; st[mt].o[i][3] *= corr[1];
        }
#pragma unroll
        for (int kk = 0; kk < NB / 16; ++kk) {
            pa[mt][kk][0] = pack_bf16(s[mt][2 * kk][0], s[mt][2 * kk][1]);
            pa[mt][kk][1] = pack_bf16(s[mt][2 * kk][2], s[mt][2 * kk][3]);
            pa[mt][kk][2] = pack_bf16(s[mt][2 * kk + 1][0], s[mt][2 * kk + 1][1]);
            pa[mt][kk][3] = pack_bf16(s[mt][2 * kk + 1][2], s[mt][2 * kk + 1][3]);
        }
    }
    // O += P V: B fragments of V by transposed ldmatrix, shared by the MT tiles
#pragma unroll
    for (int kk = 0; kk < NB / 16; ++kk) {
#pragma unroll
        for (int i = 0; i < HD / 8; i += 2) {
            // matrices: (keys 16kk.., dims 8i..), (keys 16kk+8.., dims 8i..), (keys 16kk.., dims 8i+8..), (.., +8)
            unsigned b[4];
            const bf16* p = vs + (size_t)(16 * kk + (lmat & 1) * 8 + lrow) * STR + 8 * i + (lmat >> 1) * 8;
            ldmatrix_x4_trans(b, p);
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma16816(st[mt].o[i], pa[mt][kk], b[0], b[1]);
                mma16816(st[mt].o[i + 1], pa[mt][kk], b[2], b[3]);
            }
        }
    }
}

// ------------------------------------------------------------------------------------ decode
template <int HD>
__global__ void __launch_bounds__(DEC_WARPS * 32) decode_split_kernel(
    const bf16* qkv, const int* rows, const int* positions,
    const int* row_slot, const bf16* k_pages, const bf16* v_pages,
    const int* __restrict__ table, int max_blocks, int bs, int bs_shift, int nq, int nkv, float scale, int window,
    float* part_o, float* part_ml, int max_splits) {
    constexpr int STR = HD + 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // What this block needs that the kernel before it (the QKV product of this step) does not
    // write -- the row's slot and position, the page table, and every key and value older than
    // the row's own position -- is requested BEFORE waiting for that kernel; only q and the key
    // and value at the row's own position are read after the wait.
    pdl_trigger();
    const int row = rows[blockIdx.x];
    const int slot = row_slot[row];
    if (slot < 0) return;
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int pos = positions[row];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int k_first = lo + split * SPLIT_KEYS;
    if (k_first > pos) return;                               // this split holds no key of the row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int G = nq / nkv;
    const int* trow = table + (size_t)slot * max_blocks;
    constexpr int NB = HD <= 64 ? 64 : 32;                  // keys per warp iteration
    constexpr int NMMA = HD / 16;                            // tensor-core steps along the head
    constexpr int CH = HD / 8;
    bf16* vs = reinterpret_cast<bf16*>(smem_raw) + (size_t)warp * NB * STR;
    // Keys go straight from global memory into B fragments: the order of dims inside a
    // tensor-core step is free as long as q uses the same one, so lane (g, t) takes the 8
    // consecutive dims 32 p + 8 t of key g (two steps' worth) with one 16-byte load.  A last
    // odd step (head sizes 16, 48, ...) takes dims base + 4 t with an 8-byte load.
    unsigned kf[NB / 8][NMMA][2];
    auto key_row = [&](const bf16* pages, int key) -> const bf16* {
        const int blk = bs_shift >= 0 ? (key >> bs_shift) : key / bs;
        const int off = bs_shift >= 0 ? (key & (bs - 1)) : key - blk * bs;
        const int page = trow[blk];
        return page >= 0 ? pages + (((size_t)page * nkv + kvh) * bs + off) * HD : nullptr;
    };
    // (a key row that is not a whole number of 128-byte lines -- every head size but 64 and 128 --
    // shares a line with its neighbour, so these loads bypass L1: a line fetched before the wait
    // for the row before this one would hold the stale bytes of the row's own key)
    auto load_k_row = [&](int j, const bf16* krow) {         // j must be a compile-time index after unrolling
#pragma unroll
        for (int pq = 0; pq < HD / 32; ++pq) {
            uint4 v = make_uint4(0, 0, 0, 0);
            if (krow != nullptr) v = (HD % 64 == 0) ? *reinterpret_cast<const uint4*>(krow + 32 * pq + 8 * t)
                                                    : __ldcg(reinterpret_cast<const uint4*>(krow + 32 * pq + 8 * t));
            kf[j][2 * pq][0] = v.x; kf[j][2 * pq][1] = v.y;
            kf[j][2 * pq + 1][0] = v.z; kf[j][2 * pq + 1][1] = v.w;
        }
        if (HD % 32) {
            uint2 v = make_uint2(0, 0);
            if (krow != nullptr) v = __ldcg(reinterpret_cast<const uint2*>(krow + 32 * (HD / 32) + 4 * t));
            kf[j][NMMA - 1][0] = v.x; kf[j][NMMA - 1][1] = v.y;
        }
    };
    // keys key0 .. key0 + NB - 1 that are <= last_key: K into fragments, V into the shared tile
    auto load_kv = [&](int key0, int last_key) {
#pragma unroll
        for (int j = 0; j < NB / 8; ++j) {
            const int key = key0 + 8 * j + g;
            load_k_row(j, key <= last_key ? key_row(k_pages, key) : nullptr);
        }
        gather_tile<HD, NB, 32>(vs, v_pages, trow, key0, last_key + 1, bs, bs_shift, nkv, kvh, lane);
        __pipeline_commit();
    };
    const int w_first = k_first + warp * (SPLIT_KEYS / DEC_WARPS);
    if (w_first <= pos) load_kv(w_first, pos - 1);           // everything older than this step
    pdl_wait();
    // Query fragments in the keys' order of dims: row g of the tile is query head kvh * G + g.
    unsigned qf[NMMA][4];
    {
        const bf16* qrow = qkv + (size_t)row * (nq + 2 * nkv) * HD + (size_t)kvh * G * HD;
#pragma unroll
        for (int mm = 0; mm < NMMA; ++mm) {
            const int d = (mm < 2 * (HD / 32)) ? 32 * (mm >> 1) + 8 * t + 4 * (mm & 1) : 32 * (HD / 32) + 4 * t;
            qf[mm][0] = g < G ? *reinterpret_cast<const unsigned*>(qrow + (size_t)g * HD + d) : 0u;
            qf[mm][1] = g + 8 < G ? *reinterpret_cast<const unsigned*>(qrow + (size_t)(g + 8) * HD + d) : 0u;
            qf[mm][2] = g < G ? *reinterpret_cast<const unsigned*>(qrow + (size_t)g * HD + d + 2) : 0u;
            qf[mm][3] = g + 8 < G ? *reinterpret_cast<const unsigned*>(qrow + (size_t)(g + 8) * HD + d + 2) : 0u;
        }
    }
    TileState<HD> st;
    st.init();
    const int lo_r[2] = {lo, lo}, hi_r[2] = {pos, pos};
#pragma unroll 1
    for (int it = 0; it < SPLIT_KEYS / DEC_WARPS / NB; ++it) {
        const int key0 = w_first + it * NB;
        if (key0 > pos) break;                               // warp-uniform
        if (it > 0) {
            load_kv(key0, pos);
        } else if (pos < key0 + NB) {
            // the row's own key and value, written by the kernel before this one
#pragma unroll
            for (int j = 0; j < NB / 8; ++j)
                if (key0 + 8 * j + g == pos) load_k_row(j, key_row(k_pages, pos));
            __syncwarp();                                    // the zero fill of that V row is done
            const bf16* vrow = key_row(v_pages, pos);
            if (lane < CH && vrow != nullptr)
                __pipeline_memcpy_async(vs + (size_t)(pos - key0) * STR + lane * 8, vrow + lane * 8, 16);
            __pipeline_commit();
        }
        float sc[NB / 8][4];
#pragma unroll
        for (int j = 0; j < NB / 8; ++j) {
            sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.f;
#pragma unroll
            for (int mm = 0; mm < NMMA; ++mm) mma16816(sc[j], qf[mm], kf[j][mm][0], kf[j][mm][1]);
        }
        if (key0 >= lo && key0 + NB - 1 <= pos)
            softmax_pv<HD, NB, false, true>(sc, vs, key0, lo_r, hi_r, scale, st, lane);
        else
            softmax_pv<HD, NB, true, true>(sc, vs, key0, lo_r, hi_r, scale, st, lane);
        __syncwarp();                                        // the V tile is reused by the next iteration
    }
    // merge the warps' partials in warp order
    __syncthreads();                                         // all warps are done with their K/V tiles
    float* wm = reinterpret_cast<float*>(smem_raw);          // [warps][16]
    float* wl = wm + DEC_WARPS * 16;                         // [warps][16]
    float* wo = wl + DEC_WARPS * 16;                         // [warps][16][HD]
    if (t == 0) {
        wm[warp * 16 + g] = st.m[0]; wm[warp * 16 + g + 8] = st.m[1];
        wl[warp * 16 + g] = st.l[0]; wl[warp * 16 + g + 8] = st.l[1];
    }
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
        float* o0 = wo + ((size_t)warp * 16 + g) * HD + 8 * i + 2 * t;
        float* o1 = wo + ((size_t)warp * 16 + g + 8) * HD + 8 * i + 2 * t;
        o0[0] = st.o[i][0]; o0[1] = st.o[i][1];
        o1[0] = st.o[i][2]; o1[1] = st.o[i][3];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * HD && G <= 16; i += blockDim.x) {
        const int h = i / HD, d = i - h * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) M = fmaxf(M, wm[w * 16 + h]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < DEC_WARPS; ++w) {
            const float mw = wm[w * 16 + h];
            const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
            L += wl[w * 16 + h] * f;
            O += wo[((size_t)w * 16 + h) * HD + d] * f;
        }
        const size_t pi = ((size_t)blockIdx.x * nq + kvh * G + h) * max_splits + split;
        part_o[pi * HD + d] = O;
        if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
    }
}

template <int HD>
static int launch_decode(const void* qkv, void* out, const int* rows, int n_rows, const int* positions,
                         const int* row_slot, const void* k_pages, const void* v_pages, const int* table,
                         int max_blocks, int bs, int nq, int nkv, float scale, int window, float* part_o,
                         float* part_ml, int n_splits, int max_splits, cudaStream_t s) {
    constexpr int STR = HD + 8;
    size_t smem = (size_t)DEC_WARPS * (HD <= 64 ? 64 : 32) * STR * sizeof(bf16);
    const size_t merge = (size_t)DEC_WARPS * 16 * (HD + 2) * sizeof(float);
    if (merge > smem) smem = merge;
    auto kern = decode_split_kernel<HD>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    dim3 grid(n_rows, nkv, n_splits);
    const int bs_shift = (bs & (bs - 1)) == 0 ? __builtin_ctz(bs) : -1;
    int rc = launch_pdl(kern, grid, dim3(DEC_WARPS * 32), smem, s, (const bf16*)qkv, rows, positions, row_slot,
                        (const bf16*)k_pages, (const bf16*)v_pages, table, max_blocks, bs, bs_shift, nq, nkv,
                        scale * 1.4426950408889634f, window, part_o, part_ml, max_splits);
    if (rc) return rc;
    return launch_combine<HD>(n_rows, nq, n_splits, s, rows, positions, row_slot, (const float*)part_o, (const float*)part_ml,
                              (bf16*)out, window, max_splits);
}

#define DISPATCH_HD(HDV, CALL)                                                     \
    switch (HDV) {                                                                 \
        case 16: { constexpr int H_ = 16; return CALL; }                           \
        case 32: { constexpr int H_ = 32; return CALL; }                           \
        case 48: { constexpr int H_ = 48; return CALL; }                           \
        case 64: { constexpr int H_ = 64; return CALL; }                           \
        case 80: { constexpr int H_ = 80; return CALL; }                           \
        case 96: { constexpr int H_ = 96; return CALL; }                           \
        case 112: { constexpr int H_ = 112; return CALL; }                         \
        case 128: { constexpr int H_ = 128; return CALL; }                         \
        default: return ZLLM_ERR_UNSUPPORTED;                                      \
    }

// Decode rows ``rows[0..n_rows)`` of the step.  n_splits: grid size along the splits (>= the
// splits of the longest row; a captured graph passes its bucket); max_splits: stride of the
// partial buffers.  Takes head sizes 16..128 in steps of 16 and groups nq/nkv <= 16.
ZLLM_API int zllm_attention_decode_bf16(const void* qkv, void* out, const int* rows, int n_rows, const int* positions,
                                        const int* row_slot, const void* k_pages, const void* v_pages,
                                        const int* table, int max_blocks, int bs, int nq, int nkv, int hd, float scale,
                                        int window, float* part_o, float* part_ml, int n_splits, int max_splits,
                                        void* stream) {
    if (n_rows <= 0) return 0;
    if (nkv <= 0 || nq % nkv || nq / nkv > 16 || n_splits <= 0 || n_splits > max_splits || n_splits > 65535 ||
        nkv > 65535)
        return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    DISPATCH_HD(hd, (launch_decode<H_>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table,
                                       max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, max_splits,
                                       s)))
}

// ------------------------------------------------------------------------------------ prefill
// tiles [n_tiles][4] = (first row, rows (<= 128), slot, position of first row).
// NWARPS warps of MT 16-row tiles each cover the 128 query rows of a tile: head sizes up to 64
// run 4 warps x 2 tiles (K/V fragments shared by two tiles), larger ones 8 warps x 1 tile
// (the accumulators of two tiles would not fit the registers).
template <int HD, int MT, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32, MT == 2 ? 2 : 1) prefill_kernel(
    const bf16* qkv, bf16* out, const int* __restrict__ tiles,
    const bf16* k_pages, const bf16* v_pages, const int* __restrict__ table,
    int max_blocks, int bs, int bs_shift, int nq, int nkv, float scale, int window) {
    static_assert(MT * NWARPS * 16 == PF_QROWS, "the warps' tiles must cover the query tile");
    constexpr int STR = HD + 8;
    constexpr int NT = NWARPS * 32;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* kbuf = reinterpret_cast<bf16*>(smem_raw);          // [PF_STAGES][PF_KEYS][STR]
    bf16* vbuf = kbuf + PF_STAGES * PF_KEYS * STR;           // [PF_STAGES][PF_KEYS][STR]
    // heads run fastest over the grid and later tiles (which see more keys) come first: the CTAs
    // with the most work start first for ALL heads and the short ones fill the tail
    const int* tl = tiles + 4 * (gridDim.y - 1 - blockIdx.y);
    const int row0 = tl[0], n_rows = tl[1], slot = tl[2], pos0 = tl[3];
    if (n_rows <= 0 || slot < 0) return;                     // an empty tile (padding of a tile list of fixed size)
    const int h = blockIdx.x;
    const int kvh = h / (nq / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int* trow = table + (size_t)slot * max_blocks;
    const int last_pos = pos0 + n_rows - 1;                  // last key any row of the tile sees
    const int first_key = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int kb_first = first_key / PF_KEYS;
    const int kb_last = last_pos / PF_KEYS;
    const int wrow0 = warp * MT * 16;                        // first row of the warp within the tile
    unsigned qf[MT][HD / 16][4];
    TileState<HD> st[MT];
    int lo_r[MT][2], hi_r[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int r_a = wrow0 + mt * 16 + g, r_b = r_a + 8;  // rows within the tile
        const size_t stride = (size_t)(nq + 2 * nkv) * HD;
        const bf16* qa = qkv + (size_t)(row0 + r_a) * stride + (size_t)h * HD;
        const bf16* qb = qkv + (size_t)(row0 + r_b) * stride + (size_t)h * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            const int d = 16 * kk + 2 * t;
            qf[mt][kk][0] = r_a < n_rows ? *reinterpret_cast<const unsigned*>(qa + d) : 0u;
            qf[mt][kk][1] = r_b < n_rows ? *reinterpret_cast<const unsigned*>(qb + d) : 0u;
            qf[mt][kk][2] = r_a < n_rows ? *reinterpret_cast<const unsigned*>(qa + d + 8) : 0u;
            qf[mt][kk][3] = r_b < n_rows ? *reinterpret_cast<const unsigned*>(qb + d + 8) : 0u;
        }
        st[mt].init();
        hi_r[mt][0] = r_a < n_rows ? pos0 + r_a : -1;        // rows beyond the tile see nothing
        hi_r[mt][1] = r_b < n_rows ? pos0 + r_b : -1;
        lo_r[mt][0] = window > 0 ? max(0, hi_r[mt][0] - window + 1) : 0;
        lo_r[mt][1] = window > 0 ? max(0, hi_r[mt][1] - window + 1) : 0;
    }
    constexpr int WR = MT * 16;                              // rows of the warp
    const int w_hi = pos0 + min(n_rows - 1, wrow0 + WR - 1);  // last key this warp's rows see
    const int w_lo = window > 0 ? max(0, pos0 + wrow0 - window + 1) : 0;
    // the range every row of the warp sees in full (empty when the warp holds rows beyond the tile)
    const int w_min_hi = (wrow0 + WR - 1 < n_rows) ? pos0 + wrow0 : -1;
    const int w_max_lo = window > 0 ? max(0, pos0 + wrow0 + WR - 1 - window + 1) : 0;

    // three-stage ring: tiles kb + 1 and kb + 2 are in flight while tile kb is used
    auto load_tile = [&](int kb, int stage) {
        gather_tile<HD, PF_KEYS, NT>(kbuf + (size_t)stage * PF_KEYS * STR, k_pages, trow, kb * PF_KEYS, last_pos + 1,
                                     bs, bs_shift, nkv, kvh, threadIdx.x);
        gather_tile<HD, PF_KEYS, NT>(vbuf + (size_t)stage * PF_KEYS * STR, v_pages, trow, kb * PF_KEYS, last_pos + 1,
                                     bs, bs_shift, nkv, kvh, threadIdx.x);
    };
    load_tile(kb_first, 0);
    __pipeline_commit();
    if (kb_first + 1 <= kb_last) load_tile(kb_first + 1, 1);
    __pipeline_commit();
    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int cur = (kb - kb_first) % PF_STAGES;
        if (kb + 2 <= kb_last) load_tile(kb + 2, (kb - kb_first + 2) % PF_STAGES);
        __pipeline_commit();
        __pipeline_wait_prior(2);
        __syncthreads();
        const int key0 = kb * PF_KEYS;
        if (key0 <= w_hi && key0 + PF_KEYS - 1 >= w_lo) {    // warp-uniform: some key of the tile is visible
            if (key0 + PF_KEYS - 1 <= w_min_hi && key0 >= w_max_lo)   // every key visible to every row of the warp
                attend_block<HD, PF_KEYS, false, MT>(qf, kbuf + (size_t)cur * PF_KEYS * STR,
                                                     vbuf + (size_t)cur * PF_KEYS * STR, key0, lo_r, hi_r, scale, st, lane);
            else
                attend_block<HD, PF_KEYS, true, MT>(qf, kbuf + (size_t)cur * PF_KEYS * STR,
                                                    vbuf + (size_t)cur * PF_KEYS * STR, key0, lo_r, hi_r, scale, st, lane);
        }
        __syncthreads();
    }
    __pipeline_wait_prior(0);
    // normalise and store
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int r_a = wrow0 + mt * 16 + g, r_b = r_a + 8;
        const float inv0 = st[mt].l[0] > 0.f ? 1.f / st[mt].l[0] : 0.f;
        const float inv1 = st[mt].l[1] > 0.f ? 1.f / st[mt].l[1] : 0.f;
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            const int d = 8 * i + 2 * t;
            if (r_a < n_rows)
                *reinterpret_cast<unsigned*>(out + ((size_t)(row0 + r_a) * nq + h) * HD + d) =
                    pack_bf16(st[mt].o[i][0] * inv0, st[mt].o[i][1] * inv0);
            if (r_b < n_rows)
                *reinterpret_cast<unsigned*>(out + ((size_t)(row0 + r_b) * nq + h) * HD + d) =
                    pack_bf16(st[mt].o[i][2] * inv1, st[mt].o[i][3] * inv1);
        }
    }
}

template <int HD>
static int launch_prefill(const void* qkv, void* out, const int* tiles, int n_tiles, const void* k_pages,
                          const void* v_pages, const int* table, int max_blocks, int bs, int nq, int nkv, float scale,
                          int window, cudaStream_t s) {
    constexpr int STR = HD + 8;
    constexpr int MT = HD <= 64 ? 2 : 1;
    constexpr int NWARPS = PF_QROWS / (16 * MT);
    const size_t smem = (size_t)2 * PF_STAGES * PF_KEYS * STR * sizeof(bf16);
    auto kern = prefill_kernel<HD, MT, NWARPS>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    const int bs_shift = (bs & (bs - 1)) == 0 ? __builtin_ctz(bs) : -1;
    kern<<<dim3(nq, n_tiles), NWARPS * 32, smem, s>>>((const bf16*)qkv, (bf16*)out, tiles, (const bf16*)k_pages,
                                                      (const bf16*)v_pages, table, max_blocks, bs, bs_shift, nq, nkv,
                                                      scale * 1.4426950408889634f, window);
    return launch_status();
}

// tiles: [n_tiles][4] int32 (first row, rows <= 128, slot, position of the first row)
ZLLM_API int zllm_attention_prefill_bf16(const void* qkv, void* out, const int* tiles, int n_tiles,
                                         const void* k_pages, const void* v_pages, const int* table, int max_blocks,
                                         int bs, int nq, int nkv, int hd, float scale, int window, void* stream) {
    if (n_tiles <= 0) return 0;
    if (nkv <= 0 || nq % nkv || n_tiles > 65535) return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    DISPATCH_HD(hd, (launch_prefill<H_>(qkv, out, tiles, n_tiles, k_pages, v_pages, table, max_blocks, bs, nq, nkv,
                                        scale, window, s)))
}

// ------------------------------------------------------------------------------------ no-alloc variant
// The decode kernels above with their scratch in a fixed array inside the library, for callers
// that cannot allocate (see attention_noalloc.h, which has the full contract).
#include "attention_noalloc.h"
#include <stdio.h>

// Per-split partials of the last call: [rows][nq][n_splits][hd] accumulators followed by
// [rows][nq][n_splits][2] (max, sum).  In host code this name is only a handle: the device
// address comes from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_scratch[ZLLM_NOALLOC_SCRATCH_FLOATS];

#define NOALLOC_MAX_DEVICES 64
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES];     // device address of the array, per device

static void noalloc_msg(char* err, int err_len, const char* text) {
    if (err != nullptr && err_len > 0) snprintf(err, (size_t)err_len, "%s", text);
}

ZLLM_API int zllm_attention_decode_bf16_noalloc(const void* qkv, void* out, const int* rows, int n_rows,
                                                const int* positions, const int* row_slot, const void* k_pages,
                                                const void* v_pages, const int* table, int max_blocks, int bs, int nq,
                                                int nkv, int hd, float scale, int window, int n_splits, void* stream,
                                                char* err, int err_len) {
    if (n_rows <= 0) return 0;
    if (nkv <= 0 || nq <= 0 || nq % nkv || nq / nkv > 16 || n_splits <= 0 || n_splits > 65535 || nkv > 65535 ||
        hd % 16 || hd < 16 || hd > 128 || !(scale > 0.f) || bs <= 0 || max_blocks <= 0) {
        noalloc_msg(err, err_len, "attention_decode_noalloc: head size must be 16..128 in steps of 16, nq a multiple "
                                  "of nkv with at most 16 query heads per kv head, scale > 0, n_splits in 1..65535, "
                                  "page size and pages per request positive");
        return ZLLM_ERR_UNSUPPORTED;
    }
    const unsigned long long need = (unsigned long long)n_rows * nq * n_splits * (hd + 2);
    if (need > (unsigned long long)ZLLM_NOALLOC_SCRATCH_FLOATS) {
        if (err != nullptr && err_len > 0)
            snprintf(err, (size_t)err_len,
                     "attention_decode_noalloc: rows * nq * n_splits * (hd + 2) = %llu floats exceeds the built-in "
                     "scratch of %d floats; use fewer rows per call or the entry point that takes scratch buffers",
                     need, ZLLM_NOALLOC_SCRATCH_FLOATS);
        return ZLLM_NOALLOC_TOO_LARGE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { noalloc_msg(err, err_len, cudaGetErrorString(e)); return (int)e; }
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) {
        noalloc_msg(err, err_len, "attention_decode_noalloc: device index beyond 63");
        return ZLLM_ERR_UNSUPPORTED;
    }
    float* scratch = g_noalloc_ptr[dev];
    if (scratch == nullptr) {
        // once per device, with that device current: the array's address on THIS device
        e = cudaGetSymbolAddress((void**)&scratch, g_noalloc_scratch);
        if (e != cudaSuccess || scratch == nullptr) {
            noalloc_msg(err, err_len, e != cudaSuccess ? cudaGetErrorString(e) : "no address for the scratch array");
            return e != cudaSuccess ? (int)e : ZLLM_ERR_UNSUPPORTED;
        }
        g_noalloc_ptr[dev] = scratch;
    }
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)n_rows * nq * n_splits * hd;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    switch (hd) {
        case 16: rc = launch_decode<16>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
        case 32: rc = launch_decode<32>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
        case 48: rc = launch_decode<48>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
        case 64: rc = launch_decode<64>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
        case 80: rc = launch_decode<80>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
        case 96: rc = launch_decode<96>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
        case 112: rc = launch_decode<112>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
        default: rc = launch_decode<128>(qkv, out, rows, n_rows, positions, row_slot, k_pages, v_pages, table, max_blocks, bs, nq, nkv, scale, window, part_o, part_ml, n_splits, n_splits, s); break;
    }
    if (rc != 0) noalloc_msg(err, err_len, rc == ZLLM_ERR_UNSUPPORTED ? "sizes not taken by the kernel" : cudaGetErrorString((cudaError_t)rc));
    return rc;
}
