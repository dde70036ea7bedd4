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

// SiLU in float.  The 32-bit path divides and exponentiates exactly; the bfloat16 path, whose result is
// rounded to 8 bits of mantissa at once, uses the hardware's approximations (a few units in the last
// place of a float) - the same function in the SwiGLU kernel and in the matrix product's epilogue.
template <typename T> __device__ __forceinline__ float silu_f32(float g);
template <> __device__ __forceinline__ float silu_f32<float>(float g) { return g / (1.f + expf(-g)); }
template <> __device__ __forceinline__ float silu_f32<bf16>(float g) { return __fdividef(g, 1.f + __expf(-g)); }

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

// A kernel's cudaFuncAttributeMaxDynamicSharedMemorySize is a setting of the device that is current: one record
// of the largest size asked so far for each device (a function-local static per kernel instance), guarded so that
// host threads may launch side by side.  Returns 0 or the cudaError_t.
#include <mutex>
struct AcvSmemConfig {
    int bytes[64];
    std::mutex lock;
};
template <typename Kernel>
static inline int acv_ensure_smem(AcvSmemConfig& cfg, Kernel kernel, int smem) {
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= 64) return ACV_ERR_SIZE;
    std::lock_guard<std::mutex> guard(cfg.lock);
    if (smem > cfg.bytes[device]) {
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        cfg.bytes[device] = smem;
    }
    return 0;
}

// ----------------------------------------------------------------------------- programmatic dependent launch
// Kernels of the serving path may be launched so that a kernel begins while the one before it in
// the stream is still finishing: it lets its successor start at once (pdl_launch_dependents) and
// waits for its predecessor's results (pdl_wait) before it touches global memory.  What comes
// before that wait overlaps the predecessor's tail: block start-up, barrier set-up, tensor-memory
// allocation.  Launched without the attribute, both instructions do nothing.  Which kernel classes
// get the attribute is a bit set (acv_set_pdl); measured on the decode step of a Qwen3-8B shape with
// the device timeline, every class gains (the gaps of 1.7 us before the rotation and the attention
// kernels close), so all are on by default.  A kernel launched with the attribute must execute
// pdl_wait in every CTA before it reads or writes what earlier kernels touch: its own successor's
// wait covers only this kernel's completion, which therefore has to imply its predecessors'.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline int acv_pdl_flag = 0x3f;   // bit set of kernel classes launched with the attribute; acv_set_pdl changes it
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
// a float into another CTA's shared memory whose 4 bytes are counted at an mbarrier of that CTA (both addresses in the
// cluster's window): the receiver waits on its own barrier for the bytes, no barrier of the whole cluster is needed
__device__ __forceinline__ void cluster_store_f32_counted(uint32_t addr, float v, uint32_t bar) {
    asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
                 ::"r"(addr), "r"(__float_as_uint(v)), "r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_store_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
// The two halves of a cluster barrier, for a CTA that has to know that its peers have started before it
// writes into their shared memory: arrive early, wait just before the first remote store.  Every thread of
// every CTA of the cluster executes each half once per phase.
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// every thread of every CTA of the cluster passes here once (release before, acquire after)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------- timeline (diagnostic builds only)
// Compiled with -DACV_TIMELINE every instrumented kernel logs, per CTA, when it began and ended (the
// device-wide nanosecond timer), its kernel id, block, grid size and SM; single events carry an id of their
// own.  Each source file keeps its own log (no relocatable device code); acv_tl_read_<file> copies it out.
// Without the flag the macros expand to nothing.
#ifdef ACV_TIMELINE
#define ACV_TL_CAP (1 << 16)
#define ACV_TL_MARKS 12
struct AcvTlRecord { unsigned long long t0, t1; int kernel, block, grid, smid; unsigned long long mark[ACV_TL_MARKS]; unsigned long long cycles; };
static __device__ AcvTlRecord acv_tl_log[ACV_TL_CAP];
static __device__ unsigned int acv_tl_count;
__device__ __forceinline__ unsigned long long acv_tl_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// begin at construction, end at destruction; the marks of the CTA's threads wait in shared memory and the
// whole record is written once, by one thread, when the kernel ends (nothing is sent to memory before)
struct AcvTlScope {
    unsigned long long t0; long long c0; int kernel; bool mine; unsigned long long* marks;
    __device__ __forceinline__ AcvTlScope(int k, int thread, unsigned long long* m)
        : kernel(k), mine((int)threadIdx.x == thread), marks(m) {
        if (mine) {
            t0 = acv_tl_now();
            c0 = clock64();
            for (int i = 0; i < ACV_TL_MARKS; ++i) marks[i] = 0;
        }
    }
    __device__ __forceinline__ ~AcvTlScope() {
        if (!mine) return;
        const unsigned long long t1 = acv_tl_now();
        const long long c1 = clock64();        // SM cycles of the CTA's life: with t1 - t0, the clock it ran at
        const unsigned int i = atomicAdd(&acv_tl_count, 1u);
        if (i >= ACV_TL_CAP) return;
        unsigned int smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        AcvTlRecord r;
        r.t0 = t0; r.t1 = t1; r.kernel = kernel;
        r.block = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        r.grid = gridDim.x * gridDim.y * gridDim.z; r.smid = (int)smid;
        for (int k = 0; k < ACV_TL_MARKS; ++k) r.mark[k] = marks[k];
        r.cycles = (unsigned long long)(c1 - c0);
        acv_tl_log[i] = r;
    }
};
#define ACV_TL(kernel_id, thread)                                   \
    __shared__ unsigned long long acv_tl_marks[ACV_TL_MARKS];       \
    AcvTlScope acv_tl_scope(kernel_id, thread, acv_tl_marks)
#define ACV_TL_MARK(i) (acv_tl_marks[i] = acv_tl_now())             // by one thread; i < ACV_TL_MARKS
// sums of waiting times inside the loops of the matrix product (marks used as sums of nanoseconds, each by one
// thread): the timer reads cost the loops some 35 cycles each, so they are compiled only with -DACV_TIMELINE_SUMS
#ifdef ACV_TIMELINE_SUMS
#define ACV_TL_NOW() acv_tl_now()
#define ACV_TL_ADD(i, since) (acv_tl_marks[i] += acv_tl_now() - (since))
#else
#define ACV_TL_NOW() 0ull
#define ACV_TL_ADD(i, since) ((void)(since))
#endif
#define ACV_TL_EXPORT(file)                                                                                     \
    ACV_API int acv_tl_read_##file(void* host, int cap, int reset) {                                            \
        unsigned int n = 0;                                                                                     \
        if (cudaMemcpyFromSymbol(&n, acv_tl_count, sizeof(n)) != cudaSuccess) return -1;                        \
        if (n > ACV_TL_CAP) n = ACV_TL_CAP;                                                                     \
        if ((int)n > cap) n = cap;                                                                              \
        if (n && cudaMemcpyFromSymbol(host, acv_tl_log, n * sizeof(AcvTlRecord)) != cudaSuccess) return -1;     \
        if (reset) { const unsigned int z = 0; cudaMemcpyToSymbol(acv_tl_count, &z, sizeof(z)); }               \
        return (int)n;                                                                                          \
    }
#else
#define ACV_TL(kernel_id, thread)
#define ACV_TL_MARK(i)
#define ACV_TL_NOW() 0ull
#define ACV_TL_ADD(i, since) ((void)(since))
#define ACV_TL_EXPORT(file)
#endif
// kernel ids of the timeline
#define TL_GEMM 1
#define TL_NORM 2
#define TL_ROPE 3
#define TL_ATTN_DECODE 4
#define TL_ATTN_TC 5
#define TL_ATTN_CHUNK 6
#define TL_EMBED 7
#define TL_ARGMAX 8
#define TL_SWIGLU 9
// marks of the matrix product
#define TL_M_FIRST_FULL 0      // the first operand stage has landed
#define TL_M_LAST_MMA 1        // the last k-block has been issued
#define TL_M_ACC_DONE 2        // the epilogue sees the finished accumulator
#define TL_M_PART_SENT 3       // split K in a cluster: this CTA's partial tile is on its way to rank 0
#define TL_M_CLUSTER_MET 4     // ... and the cluster's CTAs have met
#define TL_M_STORED 5          // the CTA's results are written
#define TL_M_WAIT_OVER 6       // the producer's wait for the predecessor has ended
#define TL_M_STAGED 7          // split K in a cluster, rank 0: the summed tile lies in shared memory, its way out begins
// sums of nanoseconds (tokens on rows, no split of K, where marks 3 and 4 are free)
#define TL_M_SUM_STAGE_WAIT 3  // the issuing thread waited for operand stages
#define TL_M_SUM_ACC_WAIT 4    // the issuing thread waited for an accumulator buffer
#define TL_M_SUM_EPILOGUE 7    // the first epilogue thread worked on finished accumulators
#define TL_M_SUM_FREE_WAIT 8   // the loading thread waited for a stage to be free
#define TL_M_SUM_LOAD_ISSUE 9  // the loading thread issued loads
#define TL_M_SUM_MMA_ISSUE 10  // the issuing thread issued products and commits
// marks of the decode attention
#define TL_M_ATTN_LOOP_DONE 0  // a CTA's keys are done, the merge begins
