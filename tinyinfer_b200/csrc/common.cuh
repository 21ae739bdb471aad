// Shared helpers of the tinyinfer_b200 kernels (sm_100a).
// Every launcher is an extern "C" function taking raw device pointers and a stream; it returns 0
// or a non-zero code and leaves a message for ti_last_error(). Nothing here allocates.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

#define TI_API extern "C" __attribute__((visibility("default")))

enum TiDtype : int { TI_F32 = 0, TI_BF16 = 1 };

// Host side: message of the last failed call of this thread (one buffer per library).
void ti_set_error(const char* fmt, ...);
void ti_count_launch(int n = 1);

#define TI_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            ti_set_error(__VA_ARGS__);        \
            return -1;                        \
        }                                     \
    } while (0)

#define TI_CHECK_LAUNCH(name)                                                   \
    do {                                                                        \
        cudaError_t e__ = cudaGetLastError();                                   \
        if (e__ != cudaSuccess) {                                               \
            ti_set_error("%s: %s", name, cudaGetErrorString(e__));              \
            return (int)e__;                                                    \
        }                                                                       \
        ti_count_launch();                                                      \
    } while (0)

// Programmatic dependent launch: every kernel of this package waits for the kernels before it in
// the stream with ti_grid_wait() before it touches anything they wrote (and before it writes
// anything), and lets the kernel after it start its own prologue early with
// ti_grid_launch_dependents(). Launched without the attribute, both are no-ops.
__device__ __forceinline__ void ti_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ti_grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool ti_pdl_enabled();

// Launches `kernel` with the programmatic-stream-serialization attribute (unless switched off by
// TINYINFER_B200_PDL=0): it may begin while the previous kernel of the stream drains.
template <typename... KArgs, typename... Args>
cudaError_t ti_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ti_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// Sum over a block of up to 1024 threads; every thread gets the result. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarp ? red[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) red[32] = t;
    }
    __syncthreads();
    float r = red[32];
    __syncthreads();
    return r;
}
