// Fused per-head RMS norm of q and k, rotary position encoding, and the append of
// k and v to their cache pages: one launch instead of three, and k never goes
// back to memory unrotated.
//
// For each (token, head) of the stacked projection's output [T, (NH+2NKV)*D]:
//   q, k:  inv = rsqrt(mean(v^2) + eps);  a = v*inv*w           (32-bit)
//          out[i]        = a[i]*cos[i] - a[i+R/2]*sin[i]         i < R/2
//          out[i + R/2]  = a[i+R/2]*cos[i] + a[i]*sin[i]
//          one rounding at the end; dimensions >= R (partial rotary) are only normed
//          (the reference's fused kernel, acvram/kernels/acvram_kernels.cu:4397-4430)
//   q:     written back in place
//   k, v:  written to page[block_table[seq][pos / page]] at row pos % page; a page
//          index < 0 writes nothing (the reference's padding-row sentinel,
//          acvram/kernels/acvram_kernels.cu:4496)
// Pages are [num_pages, NKV, page_size, D].  Each step is optional (null weight,
// null table, null pages), so that another position encoding can run between a
// norm-only and an append-only launch.
#include "common.cuh"

#define QRA_WARPS 8

template <typename T>
__global__ void qk_norm_rope_append_kernel(T* __restrict__ qkv, int row_stride, int NH, int NKV, int D,
                                           const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                           const float* __restrict__ cos_sin, int rot, int table_rows,
                                           const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                           const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows, T* __restrict__ k_pages,
                                           T* __restrict__ v_pages, int page_size, int num_pages) {
    extern __shared__ float sm_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * QRA_WARPS + warp;
    const int t = blockIdx.x;
    if (head >= NH + 2 * NKV) return;
    float* sm = sm_all + warp * D;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * D;
    const bool is_q = head < NH;
    const bool is_k = !is_q && head < NH + NKV;
    const bool is_v = !is_q && !is_k;
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    int pos = positions[t];

    float ss = 0.f;
    for (int e = lane; e < D; e += 32) {
        const float v = to_f32(src[e]);
        sm[e] = v;
        ss += v * v;
    }
    if (w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
        __syncwarp();
        for (int e = lane; e < D; e += 32) sm[e] = sm[e] * inv * w[e];
    }
    __syncwarp();

    T* dst = nullptr;
    if (is_q) {
        dst = src;
    } else if (k_pages) {
        const int seq = seq_of_token[t];
        const int pg = block_table[(size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride + pos / page_size];
        if (pg >= 0 && pg < num_pages) {
            const int kvh = is_k ? head - NH : head - NH - NKV;
            T* base = is_k ? k_pages : v_pages;
            dst = base + (((size_t)pg * NKV + kvh) * page_size + (pos % page_size)) * D;
        }
    } else if (is_k) {
        dst = src;
    }
    if (!dst) return;

    const bool rotate = cos_sin && !is_v && pos >= 0 && pos < table_rows;
    const int half = rot >> 1;
    const float* cs = cos_sin ? cos_sin + (size_t)(rotate ? pos : 0) * rot : nullptr;
    for (int e = lane; e < D; e += 32) {
        float o = sm[e];
        if (rotate && e < rot) {
            if (e < half)
                o = sm[e] * cs[e] - sm[e + half] * cs[half + e];
            else
                o = sm[e] * cs[e - half] + sm[e - half] * cs[e];
        }
        dst[e] = from_f32<T>(o);
    }
}

// Vector form for head sizes 32, 64, 128, 256 with the whole head rotated (or no rotation): a lane holds
// D/32 neighbouring elements, loaded and stored as one vector; its rotation partner (i +- D/2) sits in
// lane ^ 16, so the exchange is one shuffle per element and no shared memory is used.
template <typename T, int VEC>
__global__ void qk_norm_rope_append_vec_kernel(T* __restrict__ qkv, int row_stride, int NH, int NKV,
                                               const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                               const float* __restrict__ cos_sin, int table_rows,
                                               const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                               const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows,
                                               T* __restrict__ k_pages, T* __restrict__ v_pages, int page_size,
                                               int num_pages) {
    constexpr int D = VEC * 32;
    struct __align__(sizeof(T) * VEC) Vec { T e[VEC]; };
    ACV_TL(TL_ROPE, 0);
    pdl_launch_dependents();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head = blockIdx.y * QRA_WARPS + warp;
    const int t = blockIdx.x;
    if (head >= NH + 2 * NKV) return;
    T* src = qkv + (size_t)t * row_stride + (size_t)head * D;
    const bool is_q = head < NH;
    const bool is_k = !is_q && head < NH + NKV;
    const bool is_v = !is_q && !is_k;
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    const int pos = positions[t];

    T* dst = nullptr;
    if (is_q) {
        dst = src;
    } else if (k_pages) {
        const int seq = seq_of_token[t];
        const int pg = block_table[(size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride + pos / page_size];
        if (pg >= 0 && pg < num_pages) {
            const int kvh = is_k ? head - NH : head - NH - NKV;
            dst = (is_k ? k_pages : v_pages) + (((size_t)pg * NKV + kvh) * page_size + (pos % page_size)) * D;
        }
    } else if (is_k) {
        dst = src;
    }
    if (!dst) return;

    const Vec in = *reinterpret_cast<const Vec*>(src + lane * VEC);
    float a[VEC];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
        a[i] = to_f32(in.e[i]);
        ss += a[i] * a[i];
    }
    if (w) {
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int i = 0; i < VEC; ++i) a[i] = a[i] * inv * w[lane * VEC + i];
    }
    const bool rotate = cos_sin && !is_v && pos >= 0 && pos < table_rows;
    Vec res;
    if (cos_sin && !is_v) {    // warp-uniform: the shuffles are executed by all lanes
        const float* cs = cos_sin + (size_t)(rotate ? pos : 0) * D;
        const int i0 = (lane & 15) * VEC;           // index of this lane's first angle
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
            const float partner = __shfl_xor_sync(0xffffffffu, a[i], 16);
            const float c = cs[i0 + i], sn = cs[D / 2 + i0 + i];
            const float o = lane < 16 ? a[i] * c - partner * sn : a[i] * c + partner * sn;
            res.e[i] = from_f32<T>(rotate ? o : a[i]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < VEC; ++i) res.e[i] = from_f32<T>(a[i]);
    }
    *reinterpret_cast<Vec*>(dst + lane * VEC) = res;
}

template <typename T, int VEC>
static void launch_qra_vec(dim3 grid, cudaStream_t stream, void* qkv, int row_stride, int NH, int NKV, const float* q_w,
                           const float* k_w, float eps, const float* cos_sin, int table_rows, const int* positions,
                           const int* seq_of_token, const int* block_table, int bt_stride, const int* bt_rows, void* k_pages, void* v_pages,
                           int page_size, int num_pages) {
    acv_launch(PDL_ROPE, qk_norm_rope_append_vec_kernel<T, VEC>, grid, QRA_WARPS * 32, 0, stream,
        (T*)qkv, row_stride, NH, NKV, q_w, k_w, eps, cos_sin, table_rows, positions, seq_of_token, block_table,
        bt_stride, bt_rows, (T*)k_pages, (T*)v_pages, page_size, num_pages);
}

ACV_API int acv_qk_norm_rope_append(void* qkv, int row_stride, int T, int NH, int NKV, int D, const float* q_w,
                                    const float* k_w, float eps, const float* cos_sin, int rot, int table_rows,
                                    const int* positions, const int* seq_of_token, const int* block_table,
                                    int bt_stride, const int* bt_rows, void* k_pages, void* v_pages, int page_size, int num_pages,
                                    int dtype, cudaStream_t stream) {
    if (T <= 0) return 0;
    if (D <= 0 || D > 1024 || (cos_sin && (rot <= 0 || rot > D || (rot & 1)))) return ACV_ERR_SIZE;
    const int heads = NH + 2 * NKV;
    dim3 grid(T, (heads + QRA_WARPS - 1) / QRA_WARPS);
    if (dtype != ACV_F32 && dtype != ACV_BF16) return ACV_ERR_DTYPE;
    // vector form when a lane's elements make an aligned vector and the whole head rotates
    const int vec = D / 32;
    const size_t esz = dtype == ACV_F32 ? 4 : 2;
    const bool vec_ok = D % 32 == 0 && (vec == 1 || vec == 2 || vec == 4 || vec == 8) && (!cos_sin || rot == D) &&
                        vec * esz <= 16 && !((uintptr_t)qkv % (vec * esz)) && !((row_stride * esz) % (vec * esz)) &&
                        (!k_pages || (!((uintptr_t)k_pages % (vec * esz)) && !((uintptr_t)v_pages % (vec * esz))));
    if (vec_ok) {
#define QRA_VEC(TT, VV)                                                                                                 \
    launch_qra_vec<TT, VV>(grid, stream, qkv, row_stride, NH, NKV, q_w, k_w, eps, cos_sin, table_rows, positions,       \
                           seq_of_token, block_table, bt_stride, bt_rows, k_pages, v_pages, page_size, num_pages)
        if (dtype == ACV_F32) {
            if (vec == 1) QRA_VEC(float, 1); else if (vec == 2) QRA_VEC(float, 2); else if (vec == 4) QRA_VEC(float, 4);
            else return ACV_ERR_SIZE;
        } else {
            if (vec == 1) QRA_VEC(bf16, 1); else if (vec == 2) QRA_VEC(bf16, 2); else if (vec == 4) QRA_VEC(bf16, 4);
            else QRA_VEC(bf16, 8);
        }
#undef QRA_VEC
        return acv_launch_status();
    }
    const size_t smem = (size_t)QRA_WARPS * D * sizeof(float);
    if (dtype == ACV_F32)
        qk_norm_rope_append_kernel<float><<<grid, QRA_WARPS * 32, smem, stream>>>(
            (float*)qkv, row_stride, NH, NKV, D, q_w, k_w, eps, cos_sin, rot, table_rows, positions, seq_of_token,
            block_table, bt_stride, bt_rows, (float*)k_pages, (float*)v_pages, page_size, num_pages);
    else if (dtype == ACV_BF16)
        qk_norm_rope_append_kernel<bf16><<<grid, QRA_WARPS * 32, smem, stream>>>(
            (bf16*)qkv, row_stride, NH, NKV, D, q_w, k_w, eps, cos_sin, rot, table_rows, positions, seq_of_token,
            block_table, bt_stride, bt_rows, (bf16*)k_pages, (bf16*)v_pages, page_size, num_pages);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

ACV_TL_EXPORT(qk_rope_append)
