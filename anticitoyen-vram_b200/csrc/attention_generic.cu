// Paged causal attention, generic form: any number of query tokens per request,
// any head size in steps of 16 up to 256, float or bfloat16 pages.  One warp per
// (query token, query head).  It is the 32-bit path of the engine and the
// fallback of the bfloat16 path for head sizes the tensor-core kernels do not take.
//
// Query-head h reads kv-head h / (NH/NKV) (acvram/engine/layers.py:1012-1017).
// The keys of the step's own tokens are already in the pages, so the query at
// absolute position p sees the keys j <= p, and with a window w > 0 only
// j > p - w (mask aligned to absolute positions, acvram/engine/layers.py:1020-1041).
// s = scale * q.k; softmax over the visible keys with a running maximum and sum in
// 32-bit (acvram/kernels/acvram_kernels.cu:993-1146 has the same recurrence).
#include "common.cuh"

#define AG_WARPS 4

template <typename T, int NR>
__global__ void attn_generic_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                                    const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                    const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows, int NH, int NKV, int D,
                                    int page_size, int num_pages, float scale, int window) {
    extern __shared__ float sm_all[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y * AG_WARPS + warp;
    const int t = blockIdx.x;
    if (h >= NH) return;
    float* qs = sm_all + warp * D;
    const int kvh = h / (NH / NKV);
    const int p = positions[t];
    const int seq = seq_of_token[t];
    const int* bt = block_table + (size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride;
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * D;
    for (int e = lane; e < D; e += 32) qs[e] = to_f32(qrow[e]) * scale;
    __syncwarp();

    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.f;
    float m = -INFINITY, l = 0.f;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;

    for (int j0 = lo; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        bool valid = j <= p;
        long long row = 0;
        if (valid) {
            const int pg = bt[j / page_size];
            valid = pg >= 0 && pg < num_pages;
            row = (((long long)pg * NKV + kvh) * page_size + (j % page_size)) * D;
        }
        float s = -INFINITY;
        if (valid) {
            const T* kr = k_pages + row;
            float dot = 0.f;
            for (int e = 0; e < D; ++e) dot = fmaf(qs[e], to_f32(kr[e]), dot);
            s = dot;
        }
        const float tmax = warp_max(s);
        if (tmax == -INFINITY) continue;  // uniform: no readable key in this tile
        const float m_new = fmaxf(m, tmax);
        const float alpha = expf(m - m_new);
        const float pl = valid ? expf(s - m_new) : 0.f;
        l = l * alpha + warp_sum(pl);
        m = m_new;
#pragma unroll
        for (int r = 0; r < NR; ++r) acc[r] *= alpha;
        const int n_in_tile = min(32, p - j0 + 1);
        for (int kk = 0; kk < n_in_tile; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, pl, kk);
            const long long ro = __shfl_sync(0xffffffffu, row, kk);
            if (pk == 0.f) continue;
            const T* vr = v_pages + ro;
#pragma unroll
            for (int r = 0; r < NR; ++r) {
                const int e = lane + 32 * r;
                if (e < D) acc[r] = fmaf(pk, to_f32(vr[e]), acc[r]);
            }
        }
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * D;
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int r = 0; r < NR; ++r) {
        const int e = lane + 32 * r;
        if (e < D) orow[e] = from_f32<T>(acc[r] * inv_l);
    }
}

template <typename T>
static int launch_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                          const void* v_pages, const int* positions, const int* seq_of_token, const int* block_table,
                          int bt_stride, const int* bt_rows, int T_tokens, int NH, int NKV, int D, int page_size, int num_pages,
                          float scale, int window, cudaStream_t stream) {
    dim3 grid(T_tokens, (NH + AG_WARPS - 1) / AG_WARPS);
    const size_t smem = (size_t)AG_WARPS * D * sizeof(float);
    const int nr = (D + 31) / 32;
#define AG_CASE(N)                                                                                                   \
    case N:                                                                                                          \
        attn_generic_kernel<T, N><<<grid, AG_WARPS * 32, smem, stream>>>(                                            \
            (const T*)q, q_stride, (T*)out, out_stride, (const T*)k_pages, (const T*)v_pages, positions,             \
            seq_of_token, block_table, bt_stride, bt_rows, NH, NKV, D, page_size, num_pages, scale, window);                  \
        break;
    switch (nr) {
        AG_CASE(1) AG_CASE(2) AG_CASE(3) AG_CASE(4) AG_CASE(5) AG_CASE(6) AG_CASE(7) AG_CASE(8)
        default: return ACV_ERR_SIZE;
    }
#undef AG_CASE
    return acv_launch_status();
}

ACV_API int acv_attention_generic(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                  const void* v_pages, const int* positions, const int* seq_of_token,
                                  const int* block_table, int bt_stride, const int* bt_rows, int T_tokens, int NH, int NKV, int D,
                                  int page_size, int num_pages, float scale, int window, int dtype,
                                  cudaStream_t stream) {
    if (T_tokens <= 0) return 0;
    if (D <= 0 || D > 256 || NKV <= 0 || NH % NKV) return ACV_ERR_SIZE;
    if (dtype == ACV_F32)
        return launch_generic<float>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token,
                                     block_table, bt_stride, bt_rows, T_tokens, NH, NKV, D, page_size, num_pages, scale, window,
                                     stream);
    if (dtype == ACV_BF16)
        return launch_generic<bf16>(q, q_stride, out, out_stride, k_pages, v_pages, positions, seq_of_token,
                                    block_table, bt_stride, bt_rows, T_tokens, NH, NKV, D, page_size, num_pages, scale, window,
                                    stream);
    return ACV_ERR_DTYPE;
}
