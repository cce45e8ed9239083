// Shared by every kernel file: element types, conversions, reductions and the
// C calling convention of the launchers.
//
// Every launcher is `extern "C"`, takes raw device pointers and a stream,
// allocates nothing, and returns the cudaError_t of its launch as an int
// (0 = launched).  Element types are passed as codes so that one symbol serves
// the bfloat16 path and the true 32-bit path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

#define FL_API extern "C" __attribute__((visibility("default")))

enum FlDtype : int { FL_F32 = 0, FL_BF16 = 1 };

typedef __nv_bfloat16 bf16;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// Runs `...` with T bound to the element type of `code`; unknown codes make the
// launcher return cudaErrorInvalidValue.
#define FL_DISPATCH(code, T, ...)                                   \
    switch (code) {                                                 \
        case FL_F32: { using T = float; __VA_ARGS__; } break;       \
        case FL_BF16: { using T = bf16; __VA_ARGS__; } break;       \
        default: return (int)cudaErrorInvalidValue;                 \
    }

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

// Block-wide sum / max for blocks of up to 1024 threads (a multiple of 32).
// `scratch` is 32 floats of shared memory; every thread gets the result.  The
// order of additions depends only on the block size, so equal rows give equal
// results wherever they sit in a batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();                      // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = (lane < nwarps) ? scratch[lane] : 0.0f;
    return warp_sum(r);
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float r = (lane < nwarps) ? scratch[lane] : -CUDART_INF_F;
    return warp_max(r);
}

static inline int fl_launch_status() { return (int)cudaGetLastError(); }

// ---- programmatic dependent launch
// Kernels of a step run back to back on one stream, most of them for a few
// microseconds.  Launched with the programmatic-serialization attribute, a
// kernel may be scheduled while its predecessor is still running; it executes
// `pdl_wait()` before it touches anything the predecessor wrote (the wait
// returns once the predecessor has completed and its writes are visible), and
// `pdl_trigger()` tells the scheduler that the successor may be brought in.
// What a kernel does before its wait (barrier set-up, fetching weights that no
// kernel writes) overlaps the predecessor's tail.  FASTLLM_B200_PDL=0 turns the
// attribute off; the two instructions are then no-ops.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <stdlib.h>
static inline bool fl_pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* v = getenv("FASTLLM_B200_PDL");
        on = (v != nullptr && v[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

template <typename... KArgs, typename... Args>
static inline int fl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = fl_pdl_enabled() ? 1 : 0;
    return (int)cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
