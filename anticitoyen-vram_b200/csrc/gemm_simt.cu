// C[M,N] = A[M,K] . W[N,K]^T on the CUDA cores, accumulated in true 32-bit
// (FFMA; no tensor-core mode, hence no TF32 anywhere).  It is the matrix product
// of the 32-bit path of the model, and it computes logits in float from bfloat16
// operands (the reference upcasts the head's input and accumulates and returns
// float32, acvram/engine/model.py:369-410; products of bfloat16 values are exact
// in float, so float accumulation of bfloat16 operands is that computation).
//
// Each output element is a sum over k in ascending order within fixed 16-wide
// slabs, whatever M is: a row's result does not depend on the other rows.
#include "common.cuh"

#define GS_BM 64
#define GS_BN 64
#define GS_BK 16

template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ A, int lda, const TI* __restrict__ W, int ldw, TO* __restrict__ C, int ldc,
                 int M, int N, int K) {
    __shared__ float As[GS_BK][GS_BM + 4];
    __shared__ float Ws[GS_BK][GS_BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * GS_BM, n0 = blockIdx.x * GS_BN;
    const int tx = tid & 15, ty = tid >> 4;  // 16 x 16 threads, each a 4 x 4 micro-tile
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += GS_BK) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int idx = tid + it * 256;  // 0 .. 1023
            const int r = idx >> 4, kk = idx & 15;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
            As[kk][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
            Ws[kk][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GS_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn < N) C[(size_t)gm * ldc + gn] = from_f32<TO>(acc[i][j]);
        }
    }
}

// in_dtype: type of A and W; out_dtype: type of C.
ACV_API int acv_gemm_simt(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K,
                          int in_dtype, int out_dtype, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0) return ACV_ERR_SIZE;
    dim3 grid((N + GS_BN - 1) / GS_BN, (M + GS_BM - 1) / GS_BM);
    if (grid.y > 65535) return ACV_ERR_SIZE;
    if (in_dtype == ACV_F32 && out_dtype == ACV_F32)
        gemm_simt_kernel<float, float><<<grid, 256, 0, stream>>>((const float*)A, lda, (const float*)W, ldw, (float*)C, ldc, M, N, K);
    else if (in_dtype == ACV_BF16 && out_dtype == ACV_F32)
        gemm_simt_kernel<bf16, float><<<grid, 256, 0, stream>>>((const bf16*)A, lda, (const bf16*)W, ldw, (float*)C, ldc, M, N, K);
    else if (in_dtype == ACV_BF16 && out_dtype == ACV_BF16)
        gemm_simt_kernel<bf16, bf16><<<grid, 256, 0, stream>>>((const bf16*)A, lda, (const bf16*)W, ldw, (bf16*)C, ldc, M, N, K);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}
