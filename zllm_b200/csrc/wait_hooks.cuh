// What the kernels with bounded mbarrier waits share: the wait limit, the error word a wait sets
// when it gives up, a mirror of that word in pinned host memory (so that the host notices
// without a copy), and a hook for tests.
//
//   ZLLM_WAIT_STATE(tc, 1u << 24)          in a .cu file defines
//     c_tc_limit      polls a wait may take (tests lower it)
//     c_tc_skip       tests: the kernel's producer issues no copy at all, so that every wait for
//                     data runs out with nothing in flight and the kernel's give-up path runs
//     g_tc_error      0, or 1 + the index of the wait that gave up first
//     tc_give_up(i)   records it (device word and host mirror)
//   ZLLM_WAIT_EXPORTS(tc, gemm_tc)         defines the exported
//     zllm_gemm_tc_error()                 reads and clears the word
//     zllm_gemm_tc_set_error_mirror(p)     p: device-visible address of a pinned host int (or null)
//     zllm_gemm_tc_test_hook(limit, skip)  limit 0: the default
//
// A kernel whose wait gave up returns by itself: it stops issuing work, waits (bounded again)
// for the copies it has in flight, frees its tensor memory; its output is invalid.
#pragma once
#include "common.cuh"

#define ZLLM_WAIT_STATE(PFX, DEFAULT_LIMIT)                                                        \
    __constant__ unsigned c_##PFX##_limit = (DEFAULT_LIMIT);                                       \
    __constant__ int c_##PFX##_skip = 0;                                                           \
    __device__ int g_##PFX##_error = 0;                                                            \
    __device__ int* g_##PFX##_mirror = nullptr;                                                    \
    static const unsigned k_##PFX##_default_limit = (DEFAULT_LIMIT);                               \
    __device__ __noinline__ void PFX##_give_up(int where) {                                        \
        if (atomicCAS(&g_##PFX##_error, 0, 1 + where) == 0) {                                      \
            int* m = g_##PFX##_mirror;                                                             \
            if (m != nullptr) {                                                                    \
                *reinterpret_cast<volatile int*>(m) = 1 + where;                                   \
                __threadfence_system();                                                            \
            }                                                                                      \
        }                                                                                          \
    }

#define ZLLM_WAIT_EXPORTS(PFX, NAME)                                                               \
    ZLLM_API int zllm_##NAME##_error(void) {                                                       \
        int v = 0, zero = 0;                                                                       \
        if (cudaMemcpyFromSymbol(&v, g_##PFX##_error, sizeof(int)) != cudaSuccess) return -1;      \
        if (v) cudaMemcpyToSymbol(g_##PFX##_error, &zero, sizeof(int));                            \
        return v;                                                                                  \
    }                                                                                              \
    ZLLM_API int zllm_##NAME##_set_error_mirror(int* host_word) {                                  \
        return (int)cudaMemcpyToSymbol(g_##PFX##_mirror, &host_word, sizeof(int*));                \
    }                                                                                              \
    ZLLM_API int zllm_##NAME##_test_hook(unsigned limit, int skip_loads) {                         \
        const unsigned l = limit ? limit : k_##PFX##_default_limit;                                \
        cudaError_t e = cudaMemcpyToSymbol(c_##PFX##_limit, &l, sizeof(unsigned));                 \
        if (e == cudaSuccess) e = cudaMemcpyToSymbol(c_##PFX##_skip, &skip_loads, sizeof(int));    \
        return (int)e;                                                                             \
    }
