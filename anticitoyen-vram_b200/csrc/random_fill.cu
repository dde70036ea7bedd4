// Seeded random tensors made on the device, bit-equal to the host's version of the same arithmetic
// (acvram_b200/weights/random_init.py), so that a (seed, tensor name) pair gives the same values wherever
// they are made.  The reference has no random-weights mode in its engine; its tests write seeded
// checkpoints with torch.randn on the CPU (tests/conftest.py:141-183).
//
// Element i takes word i % 4 of Philox-4x32-10 (Salmon et al., SC'11) keyed by the tensor's 64-bit seed
// with counter i / 4.  A normal deviate is the inverse CDF of the word, piecewise linear between tabulated
// quantiles: the top bit is the sign, the next 10 bits choose one of 1024 equal-probability intervals of
// the half-normal, the remaining 21 bits interpolate inside it; the last interval (|z| > 3.3) is cut the
// same way once more by its own table (10 bits, 11 bits of interpolation).  Only rounded float additions
// and multiplications are used (no fused multiply-add, no library function), which is what makes the host
// and the device agree to the bit.  value = mean + std * z, rounded once to the output type.
#include "common.cuh"

__device__ __forceinline__ void philox4(uint64_t seed, uint64_t counter, uint32_t (&w)[4]) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    uint32_t c0 = (uint32_t)counter, c1 = (uint32_t)(counter >> 32), c2 = 0, c3 = 0;
    uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
        const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
        const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += W0; k1 += W1;
    }
    w[0] = c0; w[1] = c1; w[2] = c2; w[3] = c3;
}

__device__ __forceinline__ float normal_of_word(uint32_t w, const float* __restrict__ t1, const float* __restrict__ t2) {
    const uint32_t r = w & 0x7fffffffu, i = r >> 21;
    float a, b, frac;
    if (i < 1023u) {
        a = t1[i]; b = t1[i + 1];
        frac = __fmul_rn((float)(r & 0x1fffffu), 4.76837158203125e-07f);      // 2^-21, exact
    } else {
        const uint32_t j = (r >> 11) & 1023u;
        a = t2[j]; b = t2[j + 1];
        frac = __fmul_rn((float)(r & 0x7ffu), 4.8828125e-04f);                // 2^-11, exact
    }
    const float m = __fadd_rn(a, __fmul_rn(__fsub_rn(b, a), frac));
    return (w >> 31) ? -m : m;
}

template <typename T>
__global__ void random_normal_kernel(T* __restrict__ out, long long n, uint64_t seed, float mean, float std,
                                     const float* __restrict__ t1, const float* __restrict__ t2) {
    const long long blocks = (n + 3) >> 2;
    for (long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x; b < blocks; b += (long long)gridDim.x * blockDim.x) {
        uint32_t w[4];
        philox4(seed, (uint64_t)b, w);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long i = 4 * b + k;
            if (i < n) out[i] = from_f32<T>(__fadd_rn(mean, __fmul_rn(std, normal_of_word(w[k], t1, t2))));
        }
    }
}

__global__ void random_int_kernel(int* __restrict__ out, long long n, uint64_t seed, uint32_t mask) {
    const long long blocks = (n + 3) >> 2;
    for (long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x; b < blocks; b += (long long)gridDim.x * blockDim.x) {
        uint32_t w[4];
        philox4(seed, (uint64_t)b, w);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const long long i = 4 * b + k;
            if (i < n) out[i] = (int)(w[k] & mask);
        }
    }
}

static int fill_grid(long long n) {
    const long long want = ((n + 3) / 4 + 255) / 256;
    return (int)(want < 1 ? 1 : (want > 148 * 16 ? 148 * 16 : want));
}

// out[i] = mean + std * z_i.  t1: 1024 floats, t2: 1025 floats (the quantile tables, made by the host).
ACV_API int acv_random_normal(void* out, long long n, unsigned long long seed, float mean, float std, const float* t1,
                              const float* t2, int dtype, cudaStream_t stream) {
    if (n <= 0) return 0;
    if (dtype == ACV_F32)
        random_normal_kernel<float><<<fill_grid(n), 256, 0, stream>>>((float*)out, n, seed, mean, std, t1, t2);
    else if (dtype == ACV_BF16)
        random_normal_kernel<bf16><<<fill_grid(n), 256, 0, stream>>>((bf16*)out, n, seed, mean, std, t1, t2);
    else
        return ACV_ERR_DTYPE;
    return acv_launch_status();
}

// out[i] = word_i & mask (int32)
ACV_API int acv_random_int(int* out, long long n, unsigned long long seed, unsigned int mask, cudaStream_t stream) {
    if (n <= 0) return 0;
    random_int_kernel<<<fill_grid(n), 256, 0, stream>>>(out, n, seed, mask);
    return acv_launch_status();
}
