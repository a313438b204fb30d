// Shared declarations of the CUDA sources: dtype codes, conversions, reductions
// with a fixed order, and the error convention of the C entry points.
//
// Every entry point is `extern "C" int lp_*(...)`: 0 on success, a positive
// cudaError_t when a launch failed, -1 when the arguments were refused; the
// text of the last refusal or failure is kept per library (lp_last_error).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define LP_F32 0
#define LP_BF16 1

#ifndef LP_ERROR_DEFINED
#define LP_ERROR_DEFINED
static char lp_error_text[512] = "";
extern "C" const char* lp_last_error() { return lp_error_text; }
#endif

#define LP_REFUSE(...)                                            \
    do {                                                          \
        snprintf(lp_error_text, sizeof(lp_error_text), __VA_ARGS__); \
        return -1;                                                \
    } while (0)

static inline int lp_check_launch(const char* what) {
    cudaError_t err = cudaGetLastError();
    if (err != cudaSuccess) {
        snprintf(lp_error_text, sizeof(lp_error_text), "%s: %s", what, cudaGetErrorString(err));
        return (int)err;
    }
    return 0;
}

// ---------------------------------------------------------------- programmatic dependent launch
// Kernels of a step follow one another on one stream. Launched with lp_launch, a kernel may
// begin (be scheduled, set up, even prefetch what no earlier kernel writes) while its
// predecessor still runs; it must call lp_grid_wait() before it touches anything an earlier
// kernel wrote or read-modifies, and calls lp_grid_release() so that its own successor may
// start early. Every kernel waits, so completion stays transitive along the stream.
// lp_set_pdl(0), or LLMPLAYER_B200_PDL=0 in the environment when nothing was set, turns the early start off.
__device__ __forceinline__ void lp_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void lp_grid_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
#include <utility>
#ifndef LP_PDL_DEFINED
#define LP_PDL_DEFINED
static int lp_pdl_state = -1;      // -1: not decided yet (then the environment decides), 0: off, 1: on
// Switch the early start on or off for the launches of this library (the engine's options call this).
extern "C" void lp_set_pdl(int on) { lp_pdl_state = on ? 1 : 0; }
#endif
static inline bool lp_pdl_enabled() {
    if (lp_pdl_state < 0) {
        const char* v = getenv("LLMPLAYER_B200_PDL");
        lp_pdl_state = (v && v[0] == '0') ? 0 : 1;
    }
    return lp_pdl_state == 1;
}

template <bool EARLY = true, typename... KArgs, typename... Args>
static inline cudaError_t lp_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (EARLY && lp_pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(std::forward<Args>(args))...);
}
// The first kernel of a step starts only when everything before it on the stream has finished: kernels
// later in the step read the step's integers (lengths, page tables) before their own lp_grid_wait(), and
// those may have been written by the last kernel of the previous step.
template <typename... KArgs, typename... Args>
static inline cudaError_t lp_launch_first(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                          cudaStream_t stream, Args&&... args) {
    return lp_launch<false>(kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}

// Streaming multiprocessors of the current device (asked once per process).
static inline int lp_sm_count() {
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            sms <= 0)
            sms = 1;
    }
    return sms;
}

__device__ __forceinline__ float lp_to_float(float v) { return v; }
__device__ __forceinline__ float lp_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T lp_from_float(float v);
template <> __device__ __forceinline__ float lp_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 lp_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Sum over a warp: a butterfly, so every lane ends with the same value and the
// order of additions does not depend on anything but the lane count.
__device__ __forceinline__ float lp_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float lp_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats. Warp sums
// are added in warp order by every thread, so all threads get the same value.
__device__ __forceinline__ float lp_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = lp_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}
__device__ __forceinline__ float lp_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = lp_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = -INFINITY;
    for (int w = 0; w < nwarps; ++w) total = fmaxf(total, scratch[w]);
    return total;
}
