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

// ----------------------------------------------------------------------------- programmatic dependent launch
// Kernels of the serving path may be launched so that a kernel begins while the one before it in
// the stream is still finishing: it lets its successor start at once (pdl_launch_dependents) and
// waits for its predecessor's results (pdl_wait) before it touches global memory.  What comes
// before that wait overlaps the predecessor's tail: block start-up, barrier set-up, tensor-memory
// allocation.  Launched without the attribute, both instructions do nothing.  Which kernel classes
// get the attribute is a bit set (acv_set_pdl); measured on the decode step of a Qwen3-8B shape,
// the matrix product and the norm gain from it, the others do not, so those two are the default.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline int acv_pdl_flag = 0x3;   // bit set of kernel classes launched with the attribute; acv_set_pdl changes it
#define PDL_GEMM 1
#define PDL_NORM 2
#define PDL_ROPE 4
#define PDL_ATTN 8
#define PDL_ACT 16
#define PDL_MISC 32

template <typename... KArgs, typename... Args>
static inline void acv_launch_cluster(int kernel_class, dim3 cluster, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                                      size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (acv_pdl_flag & kernel_class) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster.x * cluster.y * cluster.z > 1) {     // thread-block clusters: CTAs of a cluster can write each other's shared memory
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
static inline void acv_launch(int kernel_class, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (acv_pdl_flag & kernel_class) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// ----------------------------------------------------------------------------- thread-block clusters
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address, in the cluster's shared window, of this CTA's shared address `local` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_store_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// every thread of every CTA of the cluster passes here once (release before, acquire after)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
