// Prefill attention over the paged cache on the 5th-generation tensor cores.
//
// One CTA per (tile of up to 128 query rows of a portion, query head).  Per block of 64 keys:
//   S = Q K^T      tcgen05.mma, M = 128 rows, N = 64 keys, K = head_dim, S float32 in tensor memory
//   softmax        8 warps; tcgen05.ld gives a THREAD half a row of S (lane = row), so the row
//                  maximum and sum need no shuffles, one exchange between the two threads of a
//                  row through shared memory; masking only in blocks that touch the
//                  diagonal; probabilities go to shared memory as bfloat16 in the K-major,
//                  128-byte-swizzled layout of an MMA operand
//   O += P V       tcgen05.mma, M = 128, N = head_dim, K = 64 keys, with V read in place as an
//                  MN-major operand (the cache's [position][dim] rows ARE that layout), O float32
//                  in tensor memory; O is rescaled in tensor memory only when a row's running
//                  maximum has moved by more than 2^8
// Q, and every page of K and V ([positions][64 dims] boxes of the pool's tensor map), come by
// TMA (three K/V stages).  Four warps have a role of their own: one loads keys, one loads values,
// one thread issues the S products and one the O products; mbarriers and tcgen05.commit connect
// them with the eight softmax warps.  Each role waits only for what it needs itself: S of block
// kb + 2 is issued as soon as the softmax warps have S of block kb in registers (not when they
// are done with it), and the keys of a later block never queue behind the values of an earlier
// one.  (In one warp, as two threads or half-warps, the roles starve each other: spinning
// divergent threads of a warp take turns slowly.)  Two CTAs fit on an SM (head size 64).  The
// grid runs heads fastest and the tiles with the most keys first.
// A portion that starts at position p attends the prefix 0..p-1 from the cache and its own
// rows causally; its own keys and values are already in the cache.
//
// zllm's counterpart: coopmat_flash_attn.comp with its query offset
// (src/backend/vulkan/mod.rs:1758-1777), whose math this follows.
//
// Takes head sizes 64 and 128, page sizes that are powers of two from 8 (16 for head size 128)
// to 128, no window.  The pool must hold finite numbers everywhere (it is created zeroed).
// Waits on mbarriers are bounded; a wait that runs out sets a flag the host reads.
#include "common.cuh"
#include "wait_hooks.cuh"
#include <cuda.h>
#include <math.h>
#include <string.h>

#define PT_ROWS 128
#define PT_KEYS 64                      // keys per block: S has PT_KEYS columns of tensor memory
#define PT_THREADS 384                  // warps: key loads, S issuer, 8 x softmax, value loads, O issuer
#define PT_LAZY 8.0f                     // see m_ref in the kernel
#define PT_WAIT_LIMIT (1u << 22)

ZLLM_WAIT_STATE(pt, PT_WAIT_LIMIT)

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, int where) {
    const unsigned limit = c_pt_limit;
    for (unsigned i = 0; i < limit; ++i) {
        unsigned done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    pt_give_up(where);
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

// Operand tile in shared memory, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 bytes
// apart.  K-major operands (Q, K, P): 64 elements of the contraction per row.  The MN-major
// operand (V): 64 elements of N per row, the contraction runs over the rows; ``lbo`` is the
// distance to the tile of the next 64 elements of N.
__device__ __forceinline__ unsigned long long umma_desc(unsigned saddr, unsigned lbo_bytes) {
    unsigned long long d = 0;
    d |= (unsigned long long)((saddr >> 4) & 0x3FFF);
    d |= (unsigned long long)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (unsigned long long)(1024 >> 4) << 32;
    d |= (unsigned long long)1 << 46;
    d |= (unsigned long long)2 << 61;
    return d;
}

__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(unsigned taddr, const unsigned (&r)[32]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                 "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                   "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                   "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
                 : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned pack2(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<unsigned*>(&v);
}

// tiles [n_tiles][4] = (first row, rows (<= 128), slot, position of first row)
//
// NSB buffers of S in tensor memory, NPB tiles of P and NS stages of K and V in shared memory;
// CTAS CTAs are to fit on an SM.  Block kb uses S buffer kb % NSB (its barriers are in their phase
// kb / NSB), P buffer kb % NPB and stage kb % NS.  An S buffer is free again as soon as the
// softmax warps have it in registers, so one is enough for the tensor core to compute S of block
// kb + 1 beside the softmax of block kb; O += P V of block kb runs beside the softmax of block
// kb + 1 when there are two P tiles.
template <int HD, int NSB, int NPB, int NS, int CTAS>
__global__ void __launch_bounds__(PT_THREADS, CTAS) prefill_tc_kernel(
    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
    const __grid_constant__ CUtensorMap map_v, bf16* out, const int* __restrict__ tiles,
    const int* __restrict__ table, int max_blocks, int bs, int bs_shift, int box_rows, int nq, int nkv, float scale) {
    constexpr int HALVES = HD / 64;                          // 64-element column boxes of a row
    constexpr int QHALF = PT_ROWS * 128;                     // [128 rows][64 elements], swizzled (Q, P)
    constexpr int KHALF = PT_KEYS * 128;                     // [PT_KEYS keys][64 elements], swizzled (K, V)
    constexpr int Q_BYTES = HALVES * QHALF;
    constexpr int KV_BYTES = HALVES * KHALF;
    constexpr int P_BYTES = (PT_KEYS / 64) * QHALF;          // [128 rows][PT_KEYS keys] as K-major halves of 64 keys
    constexpr int TMEM_COLS = NSB * PT_KEYS + HD <= 128 ? 128 : 256;     // S: NSB x PT_KEYS columns, O: HD columns
    static_assert(NSB * PT_KEYS + HD <= TMEM_COLS, "tensor memory");
    extern __shared__ unsigned char smem_raw[];
    const unsigned base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // Q | K ring | V ring | P tiles | barriers
    const unsigned q_tile = base, k_tiles = base + Q_BYTES, v_tiles = k_tiles + NS * KV_BYTES, p_tiles = v_tiles + NS * KV_BYTES;
    unsigned char* v_ptr = base_ptr + Q_BYTES + NS * KV_BYTES;
    unsigned char* p_ptr = base_ptr + Q_BYTES + 2 * NS * KV_BYTES;
    const unsigned bars = p_tiles + NPB * P_BYTES;
    // ring stage st = kb % NS: keys landed, values landed, keys read (S complete), values read (O += P V complete);
    // S buffer kb % NSB: S complete, S taken out of tensor memory; P buffer kb % NPB: P written
    // (O rescaled), O += P V complete
    const unsigned bar_q = bars;
    auto bar_k = [&](int st) { return bars + 8 * (1 + st); };
    auto bar_v = [&](int st) { return bars + 8 * (1 + NS + st); };
    auto bar_kfree = [&](int st) { return bars + 8 * (1 + 2 * NS + st); };
    auto bar_vfree = [&](int st) { return bars + 8 * (1 + 3 * NS + st); };
    auto bar_s = [&](int b) { return bars + 8 * (1 + 4 * NS + b); };
    auto bar_p = [&](int b) { return bars + 8 * (3 + 4 * NS + b); };
    auto bar_o = [&](int b) { return bars + 8 * (5 + 4 * NS + b); };
    auto bar_sfree = [&](int b) { return bars + 8 * (7 + 4 * NS + b); };
    volatile unsigned* tmem_slot = reinterpret_cast<volatile unsigned*>(p_ptr + NPB * P_BYTES + 8 * (9 + 4 * NS));
    float* xmax = reinterpret_cast<float*>(p_ptr + NPB * P_BYTES + 256);      // [2 sets][2 halves][128 rows] maxima, then [2 halves][128 rows] sums
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // Heads run fastest over the grid and later tiles (which see more keys) come first, so the
    // CTAs with the most work start first for ALL heads and the short ones fill the tail.
    pdl_trigger();
    const int* tl = tiles + 4 * (gridDim.y - 1 - blockIdx.y);
    const int row0 = tl[0], n_rows = tl[1], slot = tl[2], pos0 = tl[3];
    if (n_rows <= 0 || slot < 0) return;                     // an empty tile (padding of a tile list of fixed
                                                             // size): the whole CTA leaves before it owns anything
    const int h = blockIdx.x;
    const int kvh = h / (nq / nkv);
    const int* trow = table + (size_t)slot * max_blocks;
    const int last_pos = pos0 + n_rows - 1;                  // last key any row of the tile sees
    const int n_blocks = last_pos / PT_KEYS + 1;

    if (threadIdx.x == 0) {
        mbar_init(bar_q, 1);
        for (int st = 0; st < NS; ++st) {
            mbar_init(bar_k(st), 1);                         // expect_tx arrive + bytes
            mbar_init(bar_v(st), 1);
            mbar_init(bar_kfree(st), 1);                     // tcgen05.commit
            mbar_init(bar_vfree(st), 1);
        }
        for (int b = 0; b < NSB; ++b) {
            mbar_init(bar_s(b), 1);                          // tcgen05.commit
            mbar_init(bar_sfree(b), 8);                      // one arrive per softmax warp
        }
        for (int b = 0; b < NPB; ++b) {
            mbar_init(bar_p(b), 8);                          // one arrive per softmax warp
            mbar_init(bar_o(b), 1);                          // tcgen05.commit
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32((const void*)tmem_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem_s = *tmem_slot, tmem_o = tmem_s + NSB * PT_KEYS;
    // barriers, tensor memory and descriptors are ready; q, the pages and the output belong to
    // the step: nothing of them is touched before the kernel before this one has finished
    pdl_wait();

    if ((warp == 0 || warp == 2) && c_pt_skip) {
        // (tests: the producers issue no copy, every wait for data runs out with nothing in flight)
    } else if (warp == 0 || warp == 2) {
        // ---------------- TMA producers: warp 0 the key boxes, warp 2 the value boxes (16 lanes each) ----------------
        // Two warps, so each waits only for its own stages: the keys of a later block never wait
        // behind the values of an earlier one.
        if (warp == 0 && lane == 0) {
            mbar_expect_tx(bar_q, Q_BYTES);
            for (int hf = 0; hf < HALVES; ++hf)
                tma_load_2d(q_tile + hf * QHALF, &map_q, h * HD + hf * 64, row0, bar_q);
        }
        const int n_box = (PT_KEYS / box_rows) * HALVES;
        const int bidx = lane & 15, is_v = warp == 2;
        const unsigned hmask = 0xffffffffu;
        const int pb = bidx / HALVES, half = bidx - pb * HALVES;
        const unsigned box_bytes = (unsigned)box_rows * 128u;
        bool ok = true;
        for (int kb = 0; kb < n_blocks && ok; ++kb) {
            const int st = kb % NS;
            const unsigned prev = ((kb / NS) & 1) ^ 1;       // parity of the phase in which block kb - NS used the stage
            const int key_b0 = kb * PT_KEYS + pb * box_rows;
            bool valid = lane < 16 && bidx < n_box && key_b0 <= last_pos;
            int y = 0;
            if (valid) {
                const int page = trow[key_b0 >> bs_shift];
                valid = page >= 0;
                y = (page * nkv + kvh) * bs + (key_b0 & (bs - 1));
            }
            const unsigned m = __ballot_sync(hmask, valid);
            if (!is_v) {
                // keys: the stage is free when S of block kb - NS is complete
                if (kb >= NS) ok = __all_sync(hmask, mbar_wait(bar_kfree(st), prev, 0));
                if (!ok) break;
                if (lane == 0) mbar_expect_tx(bar_k(st), (unsigned)__popc(m) * box_bytes);
                __syncwarp(hmask);
                if (valid)
                    tma_load_2d(k_tiles + st * KV_BYTES + half * KHALF + pb * box_rows * 128, &map_k, half * 64, y, bar_k(st));
            } else {
                // values: the stage is free when O += P V of block kb - NS is complete
                if (kb >= NS) ok = __all_sync(hmask, mbar_wait(bar_vfree(st), prev, 1));
                if (!ok) break;
                // boxes that are not loaded must not hold garbage: probability 0 x NaN is NaN
                bool zeroed = false;
                for (int bx = 0; bx < n_box; ++bx) {
                    if ((m >> bx) & 1u) continue;
                    const int pbb = bx / HALVES, hb = bx - pbb * HALVES;
                    uint4* z = reinterpret_cast<uint4*>(v_ptr + st * KV_BYTES + hb * KHALF + pbb * box_rows * 128);
                    for (int i = lane; i < box_rows * 8; i += 32) z[i] = make_uint4(0, 0, 0, 0);
                    zeroed = true;
                }
                if (zeroed) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp(hmask);
                if (lane == 0) mbar_expect_tx(bar_v(st), (unsigned)__popc(m) * box_bytes);
                __syncwarp(hmask);
                if (valid)
                    tma_load_2d(v_tiles + st * KV_BYTES + half * KHALF + pb * box_rows * 128, &map_v, half * 64, y, bar_v(st));
            }
        }
    } else if (warp == 1 || warp == 3) {
        // ---------------- MMA issuers: warp 1 issues S = Q K^T, warp 3 issues O += P V (one lane each) ----------------
        // Two warps, so neither product waits for what only the other needs: S of block kb + 2 is
        // issued as soon as its keys have landed and the softmax warps have taken S of block kb out of
        // tensor memory; O += P V of block kb as soon as P is written and the values have landed.
        // D float32, A and B bfloat16; N >> 3 at [17,23), M >> 4 at [24,29); bit 16: B is MN-major
        if (warp == 1 && lane == 0) {
            const unsigned idesc_s = (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(PT_KEYS >> 3) << 17) |
                                     ((unsigned)(PT_ROWS >> 4) << 24);
            bool ok = mbar_wait(bar_q, 0, 2);
            for (int kb = 0; kb < n_blocks && ok; ++kb) {
                const int b = kb % NSB, st = kb % NS;
                ok = mbar_wait(bar_k(st), (kb / NS) & 1, 3);
                if (ok && kb >= NSB) ok = mbar_wait(bar_sfree(b), ((kb - NSB) / NSB) & 1, 10);   // S of block kb - NSB is in registers
                if (!ok) break;
                tc_fence_after();
                const unsigned kt = k_tiles + st * KV_BYTES;
#pragma unroll
                for (int ks = 0; ks < HD / 16; ++ks)         // 32 bytes along the head per step
                    tc_mma(tmem_s + b * PT_KEYS, umma_desc(q_tile + (ks >> 2) * QHALF + (ks & 3) * 32, 16),
                           umma_desc(kt + (ks >> 2) * KHALF + (ks & 3) * 32, 16), idesc_s, ks > 0 ? 1u : 0u);
                tc_commit(bar_s(b));
                tc_commit(bar_kfree(st));
            }
            if (!ok) {                                       // let the others run into their own limits quickly
                for (int b = 0; b < NSB; ++b) tc_commit(bar_s(b));
                for (int st = 0; st < NS; ++st) tc_commit(bar_kfree(st));
            }
        } else if (warp == 3 && lane == 0) {
            const unsigned idesc_o = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((unsigned)(HD >> 3) << 17) |
                                     ((unsigned)(PT_ROWS >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < n_blocks && ok; ++kb) {
                const int b = kb % NPB, st = kb % NS;
                ok = mbar_wait(bar_p(b), (kb / NPB) & 1, 4) && mbar_wait(bar_v(st), (kb / NS) & 1, 5);
                if (!ok) break;
                tc_fence_after();
                const unsigned pt = p_tiles + b * P_BYTES, vt = v_tiles + st * KV_BYTES;
#pragma unroll
                for (int j = 0; j < PT_KEYS / 16; ++j)       // 16 keys per step: 32 bytes of a P row, 16 rows of V
                    tc_mma(tmem_o, umma_desc(pt + (j >> 2) * QHALF + (j & 3) * 32, 16), umma_desc(vt + j * 16 * 128, KHALF),
                           idesc_o, (kb > 0 || j > 0) ? 1u : 0u);
                tc_commit(bar_o(b));
                tc_commit(bar_vfree(st));
            }
            if (!ok) {
                for (int b = 0; b < NPB; ++b) tc_commit(bar_o(b));
                for (int st = 0; st < NS; ++st) tc_commit(bar_vfree(st));
            }
        }
    } else {
        // ---------------- softmax: warps 4..11, two threads per query row ----------------
        // Warps w and w + 4 share the 32 rows of TMEM lane quadrant w & 3; ``half`` says which half
        // of a block's keys (and, for O, of the head's dims) a thread takes.  The two threads of a
        // row exchange their half-maxima through shared memory (one named barrier per quadrant).
        constexpr int HK = PT_KEYS / 2;                      // keys of a block per thread
        constexpr int HO = HD / 2;                           // dims of O per thread
        const int q = warp & 3, half = (warp - 4) >> 2;
        const int r = q * 32 + lane;                         // row of the tile = TMEM lane
        const unsigned lane_base = (unsigned)(q * 32) << 16;
        const int my_pos = pos0 + r;                         // the last key this row sees
        // m_ref: the maximum the row's exponents refer to.  It follows the true running maximum
        // only when that has moved by more than PT_LAZY (in log2 units): until then the
        // probabilities of a block are at most 2^PT_LAZY, exact in float32 sums and well inside
        // bfloat16's range, O needs no rescaling, and this block does not have to wait for the
        // products of the block before.  The final O / l is the same whatever reference was used.
        float m_ref = -INFINITY, l_run = 0.f;                // l_run: this thread's half of the row's sum
        bool ok = true;
        for (int kb = 0; kb < n_blocks; ++kb) {
            const int b = kb & 1;                            // set of the maxima's exchange buffer
            const int sb = kb % NSB, pb = kb % NPB;          // S and P buffers of the block
            const int key0 = kb * PT_KEYS + half * HK;       // first key of this thread's half
            ok = ok && mbar_wait(bar_s(sb), (kb / NSB) & 1, 6);
            tc_fence_after();
            // the row's scores of this half, once, into registers
            float sv[HK];
            {
                unsigned v[HK];
                tmem_ld32(tmem_s + sb * PT_KEYS + half * HK + lane_base, v);
#pragma unroll
                for (int i = 0; i < HK; ++i) sv[i] = __uint_as_float(v[i]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_sfree(sb));       // the buffer may be overwritten with S of block kb + NSB
            float mx = -INFINITY;
            if (kb * PT_KEYS + PT_KEYS - 1 > pos0) {         // the block reaches past the first row's own key
#pragma unroll
                for (int i = 0; i < HK; ++i) {
                    if (key0 + i > my_pos) sv[i] = -INFINITY;
                    mx = fmaxf(mx, sv[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < HK; ++i) mx = fmaxf(mx, sv[i]);
            }
            xmax[(b * 2 + half) * PT_ROWS + r] = mx;
            asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
            const float m_blk = fmaxf(mx, xmax[(b * 2 + (half ^ 1)) * PT_ROWS + r]) * scale;
            // A row decides for itself (both its threads alike); the rows of the warp that do not
            // move keep their reference and a factor of exactly 1, so a row's result does not depend
            // on its neighbours in the tile.  Rows beyond the tile's own (their scores come from
            // other requests' queries and from key boxes that were never loaded) never move.
            const bool need = r < n_rows && m_blk > m_ref + PT_LAZY;
            if (__any_sync(0xffffffffu, need)) {
                // move the reference to the true maximum and rescale l and this thread's half of O
                const float m_new = need ? fmaxf(m_ref, m_blk) : m_ref;
                const float corr = !need ? 1.f : ((m_ref == -INFINITY) ? 0.f : ex2_approx(m_ref - m_new));
                m_ref = m_new;
                l_run *= corr;
                if (kb > 0) {
                    ok = ok && mbar_wait(bar_o((kb - 1) % NPB), ((kb - 1) / NPB) & 1, 7);   // O is complete up to block kb - 1
                    tc_fence_after();
#pragma unroll 1
                    for (int c = 0; c < HO; c += 32) {
                        unsigned v[32];
                        tmem_ld32(tmem_o + lane_base + half * HO + c, v);
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                        tmem_st32(tmem_o + lane_base + half * HO + c, v);
                    }
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
            }
            const float msafe = (m_ref == -INFINITY) ? 0.f : m_ref;
            // the P buffer was last read by the products of block kb - NPB
            if (kb >= NPB) ok = ok && mbar_wait(bar_o(pb), ((kb - NPB) / NPB) & 1, 9);
            unsigned char* pt = p_ptr + pb * P_BYTES;
            float rs = 0.f;
#pragma unroll
            for (int ch = 0; ch < HK / 8; ++ch) {                            // 16-byte chunks of 8 keys
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    p[i] = ex2_approx(fmaf(sv[8 * ch + i], scale, -msafe));  // 2^(-inf) = 0 for hidden keys
                    rs += p[i];
                }
                uint4 pk;
                pk.x = pack2(p[0], p[1]);
                pk.y = pack2(p[2], p[3]);
                pk.z = pack2(p[4], p[5]);
                pk.w = pack2(p[6], p[7]);
                const int chunk = half * (HK / 8) + ch;                      // chunk of the block's PT_KEYS keys
                *reinterpret_cast<uint4*>(pt + (chunk >> 3) * QHALF + r * 128 + (((chunk & 7) ^ (r & 7)) << 4)) = pk;
            }
            l_run += rs;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the MMA reads P through the async proxy
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_p(pb));
        }
        // the finished rows: O / l as bfloat16, each thread its half of the dims
        xmax[(4 + half) * PT_ROWS + r] = l_run;
        asm volatile("bar.sync %0, 64;" ::"r"(1 + q) : "memory");
        const float l_row = l_run + xmax[(4 + (half ^ 1)) * PT_ROWS + r];
        ok = ok && mbar_wait(bar_o((n_blocks - 1) % NPB), ((n_blocks - 1) / NPB) & 1, 8);
        tc_fence_after();
        const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
#pragma unroll 1
        for (int c = 0; c < HO; c += 32) {
            unsigned v[32];
            tmem_ld32(tmem_o + lane_base + half * HO + c, v);
            if (r < n_rows && ok) {
                bf16* o = out + ((size_t)(row0 + r) * nq + h) * HD + half * HO + c;
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 pk;
                    pk.x = pack2(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
                    pk.y = pack2(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv);
                    pk.z = pack2(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv);
                    pk.w = pack2(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv);
                    *reinterpret_cast<uint4*>(o + i) = pk;
                }
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_s), "r"(TMEM_COLS) : "memory");
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

// rows x row_len bfloat16, row-major; boxes of box_rows x 64 elements, 128-byte swizzle, zero fill outside
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long row_len, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return ZLLM_ERR_UNSUPPORTED;
    cuuint64_t dims[2] = {(cuuint64_t)row_len, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)row_len * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : ZLLM_ERR_UNSUPPORTED;
}

template <int HD, int NSB, int NPB, int NS, int CTAS>
static int launch_prefill_tc(const void* qkv, int T, void* out, const int* tiles, int n_tiles, const void* k_pages,
                             const void* v_pages, long long num_pages, const int* table, int max_blocks, int bs, int nq,
                             int nkv, float scale, cudaStream_t s) {
    const int box_rows = bs < PT_KEYS ? bs : PT_KEYS;
    alignas(64) CUtensorMap mq, mk, mv;
    int e = make_map(&mq, qkv, T, (long long)(nq + 2 * nkv) * HD, PT_ROWS);
    if (e) return e;
    e = make_map(&mk, k_pages, num_pages * nkv * bs, HD, box_rows);
    if (e) return e;
    e = make_map(&mv, v_pages, num_pages * nkv * bs, HD, box_rows);
    if (e) return e;
    const size_t smem = 1024 + (size_t)(HD / 64) * (PT_ROWS + 2 * NS * PT_KEYS) * 128 +
                        NPB * (size_t)(PT_KEYS / 64) * PT_ROWS * 128 + 256 + 6 * PT_ROWS * sizeof(float);
    auto kern = prefill_tc_kernel<HD, NSB, NPB, NS, CTAS>;
    static bool attr_set = false;
    if (!attr_set) {
        cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ce != cudaSuccess) return (int)ce;
        attr_set = true;
    }
    return launch_pdl(kern, dim3(nq, n_tiles), dim3(PT_THREADS), smem, s, mq, mk, mv, (bf16*)out, tiles, table, max_blocks, bs,
                      (int)__builtin_ctz(bs), box_rows, nq, nkv, scale * 1.4426950408889634f);
}

// qkv [T][(nq + 2 nkv) hd] bfloat16 (only q is read), out [T][nq hd]; the pools [num_pages][nkv][bs][hd].
// hd 64 or 128; bs a power of two, 8..128 (16..128 for hd 128); no window.
ZLLM_API int zllm_attention_prefill_tc(const void* qkv, int T, void* out, const int* tiles, int n_tiles,
                                       const void* k_pages, const void* v_pages, long long num_pages, const int* table,
                                       int max_blocks, int bs, int nq, int nkv, int hd, float scale, void* stream) {
    if (n_tiles <= 0) return 0;
    if (nkv <= 0 || nq % nkv || n_tiles > 65535 || bs < 8 || bs > 128 || (bs & (bs - 1)) || (hd == 128 && bs < 16) ||
        (((uintptr_t)qkv | (uintptr_t)out | (uintptr_t)k_pages | (uintptr_t)v_pages) & 15))
        return ZLLM_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
#define PT_ARGS qkv, T, out, tiles, n_tiles, k_pages, v_pages, num_pages, table, max_blocks, bs, nq, nkv, scale, s
    // S buffers, P buffers, K/V stages, CTAs per SM (measured, 2,048 tokens at prefix 30,720):
    // head size 64: one S buffer and two stages 1,084 us, two and three 1,127 us; head size 128:
    // two CTAs per SM (one S, one P buffer, two stages) 2,108 us, one CTA with two and three 2,088 us
    if (hd == 64) return launch_prefill_tc<64, 1, 2, 2, 2>(PT_ARGS);
    if (hd == 128) return launch_prefill_tc<128, 2, 2, 3, 1>(PT_ARGS);
#undef PT_ARGS
    return ZLLM_ERR_UNSUPPORTED;
}



ZLLM_WAIT_EXPORTS(pt, attention_prefill_tc)
