// Building blocks of the bfloat16 attention kernels: 16-byte asynchronous copies
// into swizzled shared-memory tiles, ldmatrix fragment loads and the
// m16n8k16 bf16 tensor-core product with float accumulation.
//
// A tile is [rows][D] bfloat16, a row being D/8 chunks of 16 bytes; chunk c of row
// r is stored at chunk position (c & ~7) | ((c ^ r) & 7), so that the eight rows
// an ldmatrix reads fall into eight different banks groups.
#pragma once

#include "common.cuh"

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// byte offset of element (row, chunk) in a swizzled tile with D elements per row
template <int D>
__device__ __forceinline__ int tile_off(int row, int chunk) {
    return row * (D * 2) + (((chunk & ~7) | ((chunk ^ row) & 7)) << 4);
}

// 16-byte global -> shared copy; with valid == false the destination is zero-filled
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
    const int n = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

// d += a (16x16, row) . b (16x8, col), bf16 operands, float accumulators
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x by the hardware's approximation (relative error about 2^-22; -inf gives 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// address of key `j` of a request in a paged pool [num_pages, NKV, page_size, D]; nullptr if its page is not held
template <typename T>
__device__ __forceinline__ const T* paged_row(const T* pages, const int* bt, int j, int kvh, int NKV, int page_size,
                                              int num_pages, int D) {
    const int pg = bt[j / page_size];
    if (pg < 0 || pg >= num_pages) return nullptr;
    return pages + (((size_t)pg * NKV + kvh) * page_size + (j % page_size)) * D;
}
