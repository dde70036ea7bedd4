// Shared helpers of the sm_100a kernels: element types, conversions, reductions.
//
// Every exported launcher is plain C (no torch headers): it takes device
// pointers, sizes and a stream, launches, and returns the cudaError_t of the
// launch as an int (0 = success) or a negative code for a size it refuses.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ACV_API extern "C" __attribute__((visibility("default")))

// dtype codes shared with acvram_b200/kernels/ops.py
#define ACV_F32 0
#define ACV_BF16 1

// refusals (negative so that they cannot collide with cudaError_t values)
#define ACV_ERR_DTYPE (-2)
#define ACV_ERR_SIZE (-3)
#define ACV_ERR_ALIGN (-4)
#define ACV_ERR_SCRATCH (-5)

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// value rounded to T and read back as float: the "rounded to the model dtype" step
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f32(from_f32<T>(v)); }

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

// Sum over a block of up to 1024 threads; `red` is 32 floats of shared memory.
// Every thread gets the total.  The order of the sum is fixed by the launch
// shape only, so a row's result does not depend on the rest of the batch.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}

static inline int acv_launch_status() { return (int)cudaGetLastError(); }
