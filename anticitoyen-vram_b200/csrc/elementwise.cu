// Embedding gather, fused residual-add + RMSNorm, SwiGLU.  float and bfloat16.
//
// Rounding points follow the reference's bf16 service so that both precisions
// come from one template: the residual sum is made in 32-bit and rounded once
// (acvram/engine/couches.py:427-443); the norm's variance, rsqrt and scaling are
// 32-bit, the normalised value is rounded to the element type before the
// multiply by the weight (acvram/engine/layers.py:625-630; kernel
// acvram/kernels/acvram_kernels.cu:7922-7935); SiLU is 32-bit and rounded before
// the product with `up` (acvram/kernels/acvram_kernels.cu:8441-8452).
#include "common.cuh"

// ----------------------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ tokens, T* __restrict__ out,
                             int H, int V) {
    ACV_TL(TL_EMBED, 0);
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    int tok = tokens[t];
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);  // the host validates ids; never a bad address
    const T* src = table + (size_t)tok * H;
    T* dst = out + (size_t)t * H;
    if ((H * sizeof(T)) % 16 == 0) {
        const int n = H * sizeof(T) / 16;
        const uint4* s4 = reinterpret_cast<const uint4*>(src);
        uint4* d4 = reinterpret_cast<uint4*>(dst);
        for (int i = threadIdx.x; i < n; i += blockDim.x) d4[i] = s4[i];
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
    }
}

ACV_API int acv_embed(const void* table, const int* tokens, void* out, int T, int H, int V, int dtype,
                      cudaStream_t stream) {
    if (T <= 0) return 0;
    if (dtype == ACV_F32)
        acv_launch(PDL_MISC, embed_kernel<float>, T, 128, 0, stream, (const float*)table, tokens, (float*)out, H, V);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_MISC, embed_kernel<bf16>, T, 128, 0, stream, (const bf16*)table, tokens, (bf16*)out, H, V);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- add + RMSNorm
// One block per row.  The (summed) row is kept in shared memory as float, so the
// row is read once.  With `rows` given, block b norms row rows[b] into out[b] and
// leaves x as it is (the final norm of the rows whose logits are wanted).
template <typename T>
__global__ void add_rmsnorm_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ w,
                                   T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    extern __shared__ float row[];
    __shared__ float red[32];
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    T* xr = x + (size_t)r_in * H;
    const T* dr = delta ? delta + (size_t)r_in * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = to_f32(xr[i]);
        if (dr) {
            v = round_to<T>(v + to_f32(dr[i]));
            if (!rows) xr[i] = from_f32<T>(v);
        }
        row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)H + eps);
    T* o = out + (size_t)r_out * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = from_f32<T>(round_to<T>(row[i] * rs) * w[i]);
}

// Vector form: the row is read once with 16-byte loads and stays in registers (up to VCH chunks of
// 16 bytes per thread).  Same arithmetic and the same rounding points as the kernel above.
template <typename T, int VCH>
__global__ void add_rmsnorm_vec_kernel(T* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ w,
                                       T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    constexpr int E = 16 / sizeof(T);          // elements per 16-byte chunk
    __shared__ float red[32];
    ACV_TL(TL_NORM, 0);
    pdl_launch_dependents();
    // the norm's weights were written long before this launch: they are read while the kernel before still runs, so
    // that one round trip to memory less stands between its end and this kernel's result
    const int n_chunks = H / E;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4 wreg[VCH][E / 4];
#pragma unroll
    for (int i = 0; i < VCH; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
#pragma unroll
        for (int e4 = 0; e4 < E / 4; ++e4) wreg[i][e4] = c < n_chunks ? w4[c * (E / 4) + e4] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    const int r_out = blockIdx.x;
    const int r_in = rows ? rows[r_out] : r_out;
    uint4* xr = reinterpret_cast<uint4*>(x + (size_t)r_in * H);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + (size_t)r_in * H) : nullptr;
    float v[VCH][E];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VCH; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n_chunks) {
            uint4 xa = xr[c];
            const T* xe = reinterpret_cast<const T*>(&xa);
            if (dr) {
                uint4 da = dr[c];
                const T* de = reinterpret_cast<const T*>(&da);
                T summed[E];
#pragma unroll
                for (int e = 0; e < E; ++e) {
                    summed[e] = from_f32<T>(to_f32(xe[e]) + to_f32(de[e]));
                    v[i][e] = to_f32(summed[e]);
                }
                if (!rows) xr[c] = *reinterpret_cast<const uint4*>(summed);
            } else {
#pragma unroll
                for (int e = 0; e < E; ++e) v[i][e] = to_f32(xe[e]);
            }
#pragma unroll
            for (int e = 0; e < E; ++e) ss += v[i][e] * v[i][e];
        }
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(ss / (float)H + eps);
    uint4* o = reinterpret_cast<uint4*>(out + (size_t)r_out * H);
#pragma unroll
    for (int i = 0; i < VCH; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < n_chunks) {
            T res[E];
#pragma unroll
            for (int e4 = 0; e4 < E / 4; ++e4) {
                const float4 ww = wreg[i][e4];
                res[e4 * 4 + 0] = from_f32<T>(round_to<T>(v[i][e4 * 4 + 0] * rs) * ww.x);
                res[e4 * 4 + 1] = from_f32<T>(round_to<T>(v[i][e4 * 4 + 1] * rs) * ww.y);
                res[e4 * 4 + 2] = from_f32<T>(round_to<T>(v[i][e4 * 4 + 2] * rs) * ww.z);
                res[e4 * 4 + 3] = from_f32<T>(round_to<T>(v[i][e4 * 4 + 3] * rs) * ww.w);
            }
            o[c] = *reinterpret_cast<const uint4*>(res);
        }
    }
}

template <typename T>
static int launch_add_rmsnorm(void* x, const void* delta, const float* w, void* out, const int* rows, int n_rows,
                              int H, float eps, cudaStream_t stream) {
    constexpr int E = 16 / sizeof(T);
    const bool aligned = H % E == 0 && !((uintptr_t)x & 15) && !((uintptr_t)out & 15) && !((uintptr_t)w & 15) &&
                         (!delta || !((uintptr_t)delta & 15));
    if (aligned) {
        const int n_chunks = H / E;
        int threads = 128;
        while (threads < 1024 && threads < n_chunks) threads *= 2;
        const int per = (n_chunks + threads - 1) / threads;
        if (per <= 1) {
            acv_launch(PDL_NORM, add_rmsnorm_vec_kernel<T, 1>, n_rows, threads, 0, stream, (T*)x, (const T*)delta, w, (T*)out, rows, H, eps);
            return acv_launch_status();
        }
        if (per <= 2) {
            acv_launch(PDL_NORM, add_rmsnorm_vec_kernel<T, 2>, n_rows, threads, 0, stream, (T*)x, (const T*)delta, w, (T*)out, rows, H, eps);
            return acv_launch_status();
        }
        if (per <= 4) {
            acv_launch(PDL_NORM, add_rmsnorm_vec_kernel<T, 4>, n_rows, threads, 0, stream, (T*)x, (const T*)delta, w, (T*)out, rows, H, eps);
            return acv_launch_status();
        }
    }
    const size_t smem = (size_t)H * sizeof(float);
    if (smem > 200 * 1024) return ACV_ERR_SIZE;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int threads = H >= 4096 ? 512 : (H >= 1024 ? 256 : 128);
    add_rmsnorm_kernel<T><<<n_rows, threads, smem, stream>>>((T*)x, (const T*)delta, w, (T*)out, rows, H, eps);
    return acv_launch_status();
}

ACV_API int acv_add_rmsnorm(void* x, const void* delta, const float* w, void* out, const int* rows, int n_rows, int H,
                            float eps, int dtype, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (dtype == ACV_F32) return launch_add_rmsnorm<float>(x, delta, w, out, rows, n_rows, H, eps, stream);
    if (dtype == ACV_BF16) return launch_add_rmsnorm<bf16>(x, delta, w, out, rows, n_rows, H, eps, stream);
    return ACV_ERR_DTYPE;
}

// ----------------------------------------------------------------------------- SwiGLU
// gu is [T, 2I] (gate columns then up columns, the stacked projection's output).
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I;
        const int i = (int)(idx - t * I);
        const float g = to_f32(gu[t * 2 * I + i]);
        const float u = to_f32(gu[t * 2 * I + I + i]);
        const float s = round_to<T>(silu_f32<T>(g));
        out[idx] = from_f32<T>(s * u);
    }
}

// 16 bytes of gate and of up per thread (I a multiple of the vector width, pointers aligned)
template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, size_t total_chunks) {
    constexpr int E = 16 / sizeof(T);
    const int chunks_per_row = I / E;
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total_chunks;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / chunks_per_row;
        const int c = (int)(idx - t * chunks_per_row);
        const uint4 ga = *reinterpret_cast<const uint4*>(gu + t * 2 * I + (size_t)c * E);
        const uint4 ua = *reinterpret_cast<const uint4*>(gu + t * 2 * I + I + (size_t)c * E);
        const T* g = reinterpret_cast<const T*>(&ga);
        const T* u = reinterpret_cast<const T*>(&ua);
        T res[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float gv = to_f32(g[e]);
            res[e] = from_f32<T>(round_to<T>(silu_f32<T>(gv)) * to_f32(u[e]));
        }
        *reinterpret_cast<uint4*>(out + t * I + (size_t)c * E) = *reinterpret_cast<const uint4*>(res);
    }
}

ACV_API int acv_swiglu(const void* gu, void* out, int T, int I, int dtype, cudaStream_t stream) {
    const size_t total = (size_t)T * I;
    if (total == 0) return 0;
    {
        const int E = dtype == ACV_F32 ? 4 : 8;
        if ((dtype == ACV_F32 || dtype == ACV_BF16) && I % E == 0 && !((uintptr_t)gu & 15) && !((uintptr_t)out & 15)) {
            const size_t chunks = total / E;
            const int blocks = (int)((chunks + 255) / 256 < 148 * 16 ? (chunks + 255) / 256 : 148 * 16);
            if (dtype == ACV_F32)
                acv_launch(PDL_ACT, swiglu_vec_kernel<float>, blocks, 256, 0, stream, (const float*)gu, (float*)out, I, chunks);
            else
                acv_launch(PDL_ACT, swiglu_vec_kernel<bf16>, blocks, 256, 0, stream, (const bf16*)gu, (bf16*)out, I, chunks);
            return acv_launch_status();
        }
    }
    const int threads = 256;
    const int blocks = (int)((total + threads - 1) / threads < 148 * 16 ? (total + threads - 1) / threads : 148 * 16);
    if (dtype == ACV_F32)
        swiglu_kernel<float><<<blocks, threads, 0, stream>>>((const float*)gu, (float*)out, I, total);
    else if (dtype == ACV_BF16)
        swiglu_kernel<bf16><<<blocks, threads, 0, stream>>>((const bf16*)gu, (bf16*)out, I, total);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// Bit set of the kernel classes (PDL_* in common.cuh) launched with programmatic stream serialization; 0: none.
ACV_API void acv_set_pdl(int classes) { acv_pdl_flag = classes; }

ACV_TL_EXPORT(elementwise)

// ----------------------------------------------------------------------------- block tables kept on the device
// The block tables of all live requests stay on the device between steps ([rows][stride] page numbers, a row for
// each request slot); a step sends only the entries that changed since the step before, as (row, column, page)
// triples, and this kernel writes them.  An entry outside the table is skipped (the host never makes one).
__global__ void table_update_kernel(int* __restrict__ table, int rows, int stride, const int* __restrict__ updates, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int row = updates[3 * i], col = updates[3 * i + 1], page = updates[3 * i + 2];
    if (row >= 0 && row < rows && col >= 0 && col < stride) table[(size_t)row * stride + col] = page;
}

ACV_API int acv_table_update(int* table, int rows, int stride, const int* updates, int n, cudaStream_t stream) {
    if (n <= 0) return 0;
    table_update_kernel<<<(n + 255) / 256, 256, 0, stream>>>(table, rows, stride, updates, n);
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- bias of a projection
// out[t][n] += bias[n], the sum in float and rounded once to the element type.  The reference adds a bias where the
// weight file holds one (acvram/engine/loader.py:269-270); Qwen3's files hold none.
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ out, int ld, const float* __restrict__ bias, int rows, int N) {
    pdl_launch_dependents();
    pdl_wait();
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)rows * N) return;
    const int t = (int)(i / N), n = (int)(i - (long long)t * N);
    T* p = out + (size_t)t * ld + n;
    *p = from_f32<T>(to_f32(*p) + bias[n]);
}

ACV_API int acv_add_bias(void* out, int ld, const float* bias, int rows, int N, int dtype, cudaStream_t stream) {
    if (rows <= 0 || N <= 0) return 0;
    const long long total = (long long)rows * N;
    const unsigned grid = (unsigned)((total + 255) / 256);
    if (dtype == ACV_F32)
        acv_launch(PDL_MISC, add_bias_kernel<float>, grid, 256, 0, stream, (float*)out, ld, bias, rows, N);
    else if (dtype == ACV_BF16)
        acv_launch(PDL_MISC, add_bias_kernel<bf16>, grid, 256, 0, stream, (bf16*)out, ld, bias, rows, N);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}
