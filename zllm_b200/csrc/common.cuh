// Shared helpers of the sm_100a kernels: dtype conversion, warp/block reductions,
// launch status.  Every exported launcher returns a cudaError_t as int (0 = ok);
// launchers validate sizes on the host and refuse what they cannot run with
// ZLLM_ERR_UNSUPPORTED instead of producing a wrong result.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ZLLM_ERR_UNSUPPORTED 10001   // sizes this kernel does not take; caller picks another kernel or raises
#define ZLLM_API extern "C" __attribute__((visibility("default")))

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; the order of additions is fixed by the
// thread layout only, so a row's result never depends on what else is in the batch.
__device__ __forceinline__ float block_sum(float v, float* red /* >= 33 floats */) {
    v = warp_sum(v);
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    if (lane == 0) red[w] = v;
    __syncthreads();
    if (w == 0) {
        float t = lane < nw ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}

static inline int launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch -------------------------------------------------------
// A decode step is a chain of ~100 small kernels, each waiting for the one before.  Launched
// with the programmatic-serialization attribute, a kernel may start while its predecessor is
// still running: it announces itself (pdl_trigger), does what does not depend on the
// predecessor (fetching weights), and only then waits for the predecessor's results
// (pdl_wait).  EVERY kernel launched through launch_pdl must call pdl_wait() before it reads
// or writes anything another kernel of the step touches.
// A pointer to such data must not be declared ``const T* __restrict__``: that promises the
// compiler that nobody writes the data while the kernel runs, so it may read it through the
// read-only path and move the loads to wherever it likes -- also above the wait, where the
// kernel before has not written them yet (seen with head size 80: the decode attention read
// the previous layer's q).  Only what no kernel of a step writes (weights, rotary tables,
// block tables, tile lists) keeps the qualifier.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
#include <string.h>
// ZLLM_NO_PDL=1 launches every kernel fully serialized (for measuring what the overlap buys);
// ZLLM_NO_PDL=gemm_decode,attention_bf16 only the kernels of the source files named.
static inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("ZLLM_NO_PDL");
        v = 1;
        if (e && e[0] == '1') v = 0;
        else if (e && e[0]) {
            const char* base = strrchr(__BASE_FILE__, '/');
            base = base ? base + 1 : __BASE_FILE__;
            char name[128];
            size_t n = strcspn(base, ".");
            if (n >= sizeof(name)) n = sizeof(name) - 1;
            memcpy(name, base, n);
            name[n] = 0;
            for (const char* q = e; (q = strstr(q, name)) != nullptr; q += n) {
                const char after = q[n];
                if ((q == e || q[-1] == ',') && (after == 0 || after == ',')) { v = 0; break; }
            }
        }
    }
    return v == 1;
}

template <typename... KArgs, typename... Args>
static inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
