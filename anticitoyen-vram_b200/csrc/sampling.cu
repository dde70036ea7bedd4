// On-device sampling over float32 logits [rows, V]: penalties, greedy argmax,
// temperature, top-k, min-p, top-p and the draw, one block per row.
//
// Order and meaning follow the reference (acvram/engine/sampler.py:195-256):
// penalties on the raw logits; scaled = logit / max(T, 1e-5); top-k keeps the
// values >= the k-th largest; min-p drops p < min_p * p_max; top-p drops a token
// when the mass of the tokens before it in descending order exceeds top_p (the
// token that crosses stays, so the set is never empty); the draw is from the
// softmax of what is left.  A row with temperature <= 0 takes the argmax.
//
// Nothing is sorted: the k-th value and the top-p cut are found by bisection on
// an order-preserving 32-bit key of the float, 32 counting passes each over the
// row (which stays in L2).  The reference draws with torch.multinomial from a
// global generator; here each row has a counter-based generator, Philox-4x32-10
// keyed by the request's seed with the request's step as counter, so a draw does
// not depend on what else is in the batch.  The draw is the inverse CDF over the
// kept tokens in index order.
#include "common.cuh"

#define SMP_THREADS 1024

__device__ __forceinline__ uint32_t order_key(float f) {
    const uint32_t u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ float philox_uniform(uint64_t seed, uint64_t counter) {
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
    return ((float)c0 + 0.5f) * (1.0f / 4294967296.0f);
}

// block-wide reductions over SMP_THREADS threads; all threads get the result
__device__ __forceinline__ float block_reduce_sum(float v, float* red) { return block_sum(v, red); }

__device__ __forceinline__ float block_reduce_max(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = lane < nwarp ? red[lane] : -INFINITY;
    return warp_max(t);
}

__device__ __forceinline__ int block_reduce_sum_int(int v, int* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    int t = lane < nwarp ? red[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return t;
}

// argmax with the lowest index among equal values (torch.argmax's answer)
__device__ __forceinline__ int block_argmax(const float* row, int V, float inv_temp, float* redf, int* redi) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i] * inv_temp;
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) { redf[warp] = best; redi[warp] = bi; }
    __syncthreads();
    best = lane < nwarp ? redf[lane] : -INFINITY;
    bi = lane < nwarp ? redi[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    return bi;
}

__global__ void __launch_bounds__(SMP_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out) {
    __shared__ float redf[32];
    __shared__ int redi[32];
    const int bi = block_argmax(logits + (size_t)blockIdx.x * ld, V, 1.f, redf, redi);
    if (threadIdx.x == 0) out[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;     // a row without a value above -inf (all NaN): token 0
}

// Wide rows: each row is cut into ARG_PARTS slices, one block per slice leaves (value, index) in
// scratch, and the block that arrives last at a row picks among the slices in slice order (lowest
// index among equal values, as above).  No block waits for another.
#define ARG_PARTS 16
#define ARG_MAX_ROWS 4096
static __device__ float arg_part_val[ARG_MAX_ROWS * ARG_PARTS];
static __device__ int arg_part_idx[ARG_MAX_ROWS * ARG_PARTS];
static __device__ int arg_counter[ARG_MAX_ROWS];

__global__ void __launch_bounds__(256)
argmax_split_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ out) {
    __shared__ float redf[32];
    __shared__ int redi[32];
    __shared__ int last_s;
    ACV_TL(TL_ARGMAX, 0);
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x, part = blockIdx.y;
    const int span = ((V + ARG_PARTS - 1) / ARG_PARTS + 3) & ~3;
    const int lo = part * span, hi = min(V, lo + span);
    const float* r = logits + (size_t)row * ld;
    float best = -INFINITY;
    int bi = 0x7fffffff;
    if ((((uintptr_t)r) & 15) == 0 && (lo & 3) == 0) {
        // 16-byte loads, four in flight per thread before the first comparison (the slice is short: what
        // counts is that its loads are all on their way at once)
        const int n4 = (hi - lo) >> 2;
        const float4* r4 = reinterpret_cast<const float4*>(r + lo);
        for (int c0 = threadIdx.x; c0 < n4; c0 += 4 * blockDim.x) {
            float4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int c = c0 + k * blockDim.x;
                v[k] = c < n4 ? r4[c] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = lo + 4 * (c0 + k * blockDim.x);
                if (v[k].x > best) { best = v[k].x; bi = i; }
                if (v[k].y > best) { best = v[k].y; bi = i + 1; }
                if (v[k].z > best) { best = v[k].z; bi = i + 2; }
                if (v[k].w > best) { best = v[k].w; bi = i + 3; }
            }
        }
        for (int i = lo + (n4 << 2) + threadIdx.x; i < hi; i += blockDim.x) {
            const float v = r[i];
            if (v > best) { best = v; bi = i; }
        }
    } else {
        for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
            const float v = r[i];
            if (v > best || (v == best && i < bi)) { best = v; bi = i; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    if (lane == 0) { redf[warp] = best; redi[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        best = lane < nwarp ? redf[lane] : -INFINITY;
        bi = lane < nwarp ? redi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            arg_part_val[row * ARG_PARTS + part] = best;
            arg_part_idx[row * ARG_PARTS + part] = bi;
            __threadfence();
            last_s = atomicAdd(&arg_counter[row], 1) == ARG_PARTS - 1;
        }
    }
    __syncthreads();
    if (last_s && threadIdx.x == 0) {
        __threadfence();
        float b = -INFINITY;
        int idx = 0x7fffffff;
        for (int q = 0; q < ARG_PARTS; ++q) {
            const float v = __ldcg(&arg_part_val[row * ARG_PARTS + q]);
            const int i = __ldcg(&arg_part_idx[row * ARG_PARTS + q]);
            if (v > b || (v == b && i < idx)) { b = v; idx = i; }
        }
        out[row] = idx == 0x7fffffff ? 0 : idx;
        arg_counter[row] = 0;
    }
}

ACV_API int acv_argmax(const float* logits, int ld, int rows, int V, int* out, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0) return ACV_ERR_SIZE;
    if (V >= 16384 && rows <= ARG_MAX_ROWS) {
        acv_launch(PDL_MISC, argmax_split_kernel, dim3(rows, ARG_PARTS), 256, 0, stream, logits, ld, V, out);
        return acv_launch_status();
    }
    argmax_kernel<<<rows, SMP_THREADS, 0, stream>>>(logits, ld, V, out);
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- penalties
// One thread per (row, distinct token already seen, its count).
__global__ void penalties_kernel(float* __restrict__ logits, int ld, int V, const int* __restrict__ pen_row,
                                 const int* __restrict__ pen_token, const int* __restrict__ pen_count, int n,
                                 const float* __restrict__ repetition, const float* __restrict__ presence,
                                 const float* __restrict__ frequency) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int r = pen_row[i], tok = pen_token[i];
    if (tok < 0 || tok >= V) return;
    float v = logits[(size_t)r * ld + tok];
    const float rep = repetition[r];
    if (rep != 1.f) v = v > 0.f ? v / rep : v * rep;
    v -= presence[r];
    v -= frequency[r] * (float)pen_count[i];
    logits[(size_t)r * ld + tok] = v;
}

ACV_API int acv_apply_penalties(float* logits, int ld, int V, const int* pen_row, const int* pen_token,
                                const int* pen_count, int n, const float* repetition, const float* presence,
                                const float* frequency, cudaStream_t stream) {
    if (n <= 0) return 0;
    penalties_kernel<<<(n + 255) / 256, 256, 0, stream>>>(logits, ld, V, pen_row, pen_token, pen_count, n, repetition,
                                                          presence, frequency);
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- sample
__global__ void __launch_bounds__(SMP_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
              const unsigned long long* __restrict__ seed, const unsigned long long* __restrict__ counter,
              int* __restrict__ out_token, float* __restrict__ out_logprob) {
    __shared__ float redf[32];
    __shared__ int redi[32];
    __shared__ float scan[SMP_THREADS];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float temp = temperature[r];

    if (temp <= 0.f) {  // greedy row
        int bi = block_argmax(row, V, 1.f, redf, redi);
        if (bi == 0x7fffffff) bi = 0;           // a row without a value above -inf (all NaN): token 0, as argmax_split_kernel
        float z = 0.f;
        if (out_logprob) {
            const float mx = row[bi];
            for (int i = threadIdx.x; i < V; i += blockDim.x) z += expf(row[i] - mx);
            z = block_reduce_sum(z, redf);
        }
        if (threadIdx.x == 0) {
            out_token[r] = bi;
            if (out_logprob) out_logprob[r] = -logf(z);
        }
        return;
    }

    const float inv_t = 1.f / fmaxf(temp, 1e-5f);
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i] * inv_t);
    mx = block_reduce_max(mx, redf);

    uint32_t cut = 0;  // keys >= cut are kept
    const int k = top_k[r];
    if (k > 0 && k < V) {
        uint32_t prefix = 0;
        for (int b = 31; b >= 0; --b) {
            const uint32_t cand = prefix | (1u << b);
            int cnt = 0;
            for (int i = threadIdx.x; i < V; i += blockDim.x) cnt += order_key(row[i] * inv_t) >= cand;
            cnt = block_reduce_sum_int(cnt, redi);
            if (cnt >= k) prefix = cand;
        }
        cut = prefix;
    }
    const float mp = min_p[r];
    const bool use_minp = mp > 0.f;
    // kept(i): key >= cut and (no min-p or exp(s - max) >= min_p)
    const float tp = top_p[r];
    if (tp > 0.f && tp < 1.f) {
        float z = 0.f;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float s = row[i] * inv_t;
            const float e = expf(s - mx);
            if (order_key(s) >= cut && !(use_minp && e < mp)) z += e;
        }
        z = block_reduce_sum(z, redf);
        const float limit = tp * z;
        uint32_t prefix = 0;  // the largest key value t with mass(key > t) > limit
        for (int b = 31; b >= 0; --b) {
            const uint32_t cand = prefix | (1u << b);
            float mass = 0.f;
            for (int i = threadIdx.x; i < V; i += blockDim.x) {
                const float s = row[i] * inv_t;
                const uint32_t key = order_key(s);
                const float e = expf(s - mx);
                if (key > cand && key >= cut && !(use_minp && e < mp)) mass += e;
            }
            mass = block_reduce_sum(mass, redf);
            if (mass > limit) prefix = cand;
        }
        const uint32_t cut_p = prefix + 1u;
        cut = cut_p > cut ? cut_p : cut;
    }

    // inverse CDF in index order: each thread owns a contiguous range of indices
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int lo = threadIdx.x * chunk, hi = min(V, lo + chunk);
    float local = 0.f;
    for (int i = lo; i < hi; ++i) {
        const float s = row[i] * inv_t;
        const float e = expf(s - mx);
        if (order_key(s) >= cut && !(use_minp && e < mp)) local += e;
    }
    scan[threadIdx.x] = local;
    __syncthreads();
    __shared__ float total_s;
    __shared__ int owner_s;
    __shared__ float before_s;
    if (threadIdx.x == 0) {
        float run = 0.f;
        for (int t = 0; t < (int)blockDim.x; ++t) run += scan[t];
        const float u = philox_uniform(seed[r], counter[r]);
        const float target = u * run;
        float acc = 0.f;
        int owner = -1;
        int last_nonempty = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (scan[t] > 0.f) last_nonempty = t;
            if (owner < 0 && scan[t] > 0.f && acc + scan[t] >= target) { owner = t; before_s = acc; }
            if (owner < 0) acc += scan[t];
        }
        if (owner < 0) { owner = last_nonempty; before_s = acc - scan[last_nonempty]; }
        owner_s = owner;
        total_s = run;
        redf[0] = target;
    }
    __syncthreads();
    if ((int)threadIdx.x == owner_s) {
        const float target = redf[0];
        float acc = before_s;
        int pick = -1, last_kept = -1;
        for (int i = lo; i < hi; ++i) {
            const float s = row[i] * inv_t;
            const float e = expf(s - mx);
            if (order_key(s) >= cut && !(use_minp && e < mp)) {
                last_kept = i;
                acc += e;
                if (acc >= target) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last_kept;
        out_token[r] = pick;
        if (out_logprob) out_logprob[r] = (row[pick] * inv_t - mx) - logf(total_s);
    }
}

// ----------------------------------------------------------------------------- sample, a cluster to a row
// A wide row (a vocabulary of 150 thousand) read 70 times by one block is bound by the latency of its loads: a
// second per thousand steps of eight rows.  Here the CTAs of one thread-block cluster share a row: each keeps its
// slice of the scaled logits in shared memory, so the row is read from memory once and the bisections' passes run
// on shared memory; what a pass counts is added up over the cluster through the CTAs' shared memory (every CTA
// writes its part into every CTA's table, one cluster barrier, every CTA adds the parts in rank order, so all take
// the same decision).  The arithmetic is sample_kernel's; sums are formed slice by slice.
#define SMPC_CTAS 8
#define SMPC_THREADS 1024

struct ClusterSum {
    float* parts;          // [2][SMPC_CTAS] in this CTA's shared memory
    float* warps;          // [32]
    int turn;
    uint32_t rank;
};

// every thread gets the sum over the cluster of `v` (a float; counts up to 2^24 are exact)
__device__ __forceinline__ float cluster_all_sum(ClusterSum& c, float v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) c.warps[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (int)(blockDim.x >> 5) ? c.warps[lane] : 0.f;
        t = warp_sum(t);
        if (lane < SMPC_CTAS)
            cluster_store_f32(cluster_map((uint32_t)__cvta_generic_to_shared(c.parts + c.turn * SMPC_CTAS + c.rank), lane), t);
    }
    cluster_sync_all();
    float total = 0.f;
#pragma unroll
    for (int r = 0; r < SMPC_CTAS; ++r) total += c.parts[c.turn * SMPC_CTAS + r];
    c.turn ^= 1;
    return total;
}
__device__ __forceinline__ float cluster_all_max(ClusterSum& c, float v) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_max(v);
    if (lane == 0) c.warps[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < (int)(blockDim.x >> 5) ? c.warps[lane] : -INFINITY;
        t = warp_max(t);
        if (lane < SMPC_CTAS)
            cluster_store_f32(cluster_map((uint32_t)__cvta_generic_to_shared(c.parts + c.turn * SMPC_CTAS + c.rank), lane), t);
    }
    cluster_sync_all();
    float total = -INFINITY;
#pragma unroll
    for (int r = 0; r < SMPC_CTAS; ++r) total = fmaxf(total, c.parts[c.turn * SMPC_CTAS + r]);
    c.turn ^= 1;
    return total;
}

__global__ void __launch_bounds__(SMPC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int ld, int V, int slice, const float* __restrict__ temperature,
                      const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ min_p,
                      const unsigned long long* __restrict__ seed, const unsigned long long* __restrict__ counter,
                      int* __restrict__ out_token, float* __restrict__ out_logprob) {
    extern __shared__ float sl[];               // this CTA's slice of the scaled logits, and behind it exp(logit - maximum)
    __shared__ float parts[2 * SMPC_CTAS];
    __shared__ float warps[32];
    __shared__ float scan[SMPC_THREADS];
    __shared__ float bestv[2 * SMPC_CTAS];
    __shared__ int owner_s;
    __shared__ float before_s, target_s;
    ClusterSum cs;
    cs.parts = parts; cs.warps = warps; cs.turn = 0; cs.rank = cluster_ctarank();
    const int r = blockIdx.x / SMPC_CTAS;
    const float* row = logits + (size_t)r * ld;
    const int lo = (int)cs.rank * slice, hi = min(V, lo + slice), n = max(0, hi - lo);
    const float temp = temperature[r];
    const bool greedy = temp <= 0.f;
    const float inv_t = greedy ? 1.f : 1.f / fmaxf(temp, 1e-5f);
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[lo + i] * inv_t;
        sl[i] = v;
        mx = fmaxf(mx, v);
    }
    mx = cluster_all_max(cs, mx);           // (its barriers also make the slice visible to the CTA's threads)

    if (greedy) {
        // the lowest index that holds the maximum: the smallest of the CTAs' candidates (slices are in index order)
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            if (sl[i] == mx) bi = min(bi, lo + i);
        const float first = -cluster_all_max(cs, bi == 0x7fffffff ? -INFINITY : -(float)bi);     // indices < 2^24: exact
        const int pick = first == INFINITY ? 0 : (int)first;
        float z = 0.f;
        if (out_logprob) {
            float local = 0.f;
            for (int i = threadIdx.x; i < n; i += blockDim.x) local += expf(sl[i] - mx);
            z = cluster_all_sum(cs, local);
        }
        if (cs.rank == 0 && threadIdx.x == 0) {
            out_token[r] = pick;
            if (out_logprob) out_logprob[r] = -logf(z);
        }
        return;
    }

    // the exponentials once, for all the passes that follow (a pass is bound by its instructions, of which the
    // exponential was a third: 160 -> 142 us for 8 rows of 151 936)
    float* se = sl + slice;
    for (int i = threadIdx.x; i < n; i += blockDim.x) se[i] = expf(sl[i] - mx);
    __syncthreads();
    uint32_t cut = 0;  // keys >= cut are kept
    const int k = top_k[r];
    if (k > 0 && k < V) {
        uint32_t prefix = 0;
        for (int b = 31; b >= 0; --b) {
            const uint32_t cand = prefix | (1u << b);
            int cnt = 0;
            for (int i = threadIdx.x; i < n; i += blockDim.x) cnt += order_key(sl[i]) >= cand;
            if (cluster_all_sum(cs, (float)cnt) >= (float)k) prefix = cand;
        }
        cut = prefix;
    }
    const float mp = min_p[r];
    const bool use_minp = mp > 0.f;
    const float tp = top_p[r];
    if (tp > 0.f && tp < 1.f) {
        float z = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x) {
            const float s = sl[i];
            const float e = se[i];
            if (order_key(s) >= cut && !(use_minp && e < mp)) z += e;
        }
        z = cluster_all_sum(cs, z);
        const float limit = tp * z;
        uint32_t prefix = 0;  // the largest key value t with mass(key > t) > limit
        for (int b = 31; b >= 0; --b) {
            const uint32_t cand = prefix | (1u << b);
            float mass = 0.f;
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const float s = sl[i];
                const uint32_t key = order_key(s);
                const float e = se[i];
                if (key > cand && key >= cut && !(use_minp && e < mp)) mass += e;
            }
            if (cluster_all_sum(cs, mass) > limit) prefix = cand;
        }
        const uint32_t cut_p = prefix + 1u;
        cut = cut_p > cut ? cut_p : cut;
    }

    // inverse CDF in index order: CTA by CTA, inside a CTA each thread owns a contiguous range of its slice
    const int chunk = (n + (int)blockDim.x - 1) / (int)blockDim.x;
    const int c_lo = min(n, (int)threadIdx.x * chunk), c_hi = min(n, c_lo + chunk);
    float local = 0.f;
    for (int i = c_lo; i < c_hi; ++i) {
        const float s = sl[i];
        const float e = se[i];
        if (order_key(s) >= cut && !(use_minp && e < mp)) local += e;
    }
    scan[threadIdx.x] = local;
    // every CTA learns every CTA's total (the same exchange as a sum's, read part by part)
    {
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        float v = warp_sum(local);
        if (lane == 0) warps[warp] = v;
        __syncthreads();
        if (warp == 0) {
            float tot = lane < (int)(blockDim.x >> 5) ? warps[lane] : 0.f;
            tot = warp_sum(tot);
            if (lane < SMPC_CTAS)
                cluster_store_f32(cluster_map((uint32_t)__cvta_generic_to_shared(bestv + cs.rank), lane), tot);
        }
        cluster_sync_all();
    }
    float run = 0.f;
#pragma unroll
    for (int c = 0; c < SMPC_CTAS; ++c) run += bestv[c];
    const float u = philox_uniform(seed[r], counter[r]);
    const float target = u * run;
    // the CTA in which the target falls (the last CTA with anything kept, if rounding leaves the target beyond all)
    int owner_cta = -1, last_cta = 0;
    float acc = 0.f, before_cta = 0.f;
#pragma unroll
    for (int c = 0; c < SMPC_CTAS; ++c) {
        if (bestv[c] > 0.f) last_cta = c;
        if (owner_cta < 0 && bestv[c] > 0.f && acc + bestv[c] >= target) { owner_cta = c; before_cta = acc; }
        if (owner_cta < 0) acc += bestv[c];
    }
    if (owner_cta < 0) { owner_cta = last_cta; before_cta = acc - bestv[last_cta]; }
    if ((int)cs.rank != owner_cta) return;
    if (threadIdx.x == 0) {
        float a2 = before_cta;
        int owner = -1, last_nonempty = 0;
        for (int t = 0; t < (int)blockDim.x; ++t) {
            if (scan[t] > 0.f) last_nonempty = t;
            if (owner < 0 && scan[t] > 0.f && a2 + scan[t] >= target) { owner = t; before_s = a2; }
            if (owner < 0) a2 += scan[t];
        }
        if (owner < 0) { owner = last_nonempty; before_s = a2 - scan[last_nonempty]; }
        owner_s = owner;
        target_s = target;
    }
    __syncthreads();
    if ((int)threadIdx.x == owner_s) {
        float a3 = before_s;
        int pick = -1, last_kept = -1;
        for (int i = c_lo; i < c_hi; ++i) {
            const float s = sl[i];
            const float e = se[i];
            if (order_key(s) >= cut && !(use_minp && e < mp)) {
                last_kept = i;
                a3 += e;
                if (a3 >= target_s) { pick = i; break; }
            }
        }
        if (pick < 0) pick = last_kept;
        out_token[r] = lo + pick;
        if (out_logprob) out_logprob[r] = (sl[pick] - mx) - logf(run);
    }
}

ACV_API int acv_sample(const float* logits, int ld, int rows, int V, const float* temperature, const int* top_k,
                       const float* top_p, const float* min_p, const unsigned long long* seed,
                       const unsigned long long* counter, int* out_token, float* out_logprob, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0) return ACV_ERR_SIZE;
    // wide rows: a cluster of CTAs to a row, the row's slices in their shared memory
    const int slice = ((V + SMPC_CTAS - 1) / SMPC_CTAS + 3) & ~3;
    const int smem = 2 * slice * (int)sizeof(float);
    if (V >= 16384 && V < (1 << 24) && smem <= 200 * 1024) {
        static AcvSmemConfig smem_config;
        if (int rc = acv_ensure_smem(smem_config, sample_cluster_kernel, smem)) return rc;
        acv_launch_cluster(0, dim3(SMPC_CTAS, 1, 1), sample_cluster_kernel, dim3((unsigned)rows * SMPC_CTAS), dim3(SMPC_THREADS),
                           (size_t)smem, stream, logits, ld, V, slice, temperature, top_k, top_p, min_p, seed, counter,
                           out_token, out_logprob);
        return acv_launch_status();
    }
    sample_kernel<<<rows, SMP_THREADS, 0, stream>>>(logits, ld, V, temperature, top_k, top_p, min_p, seed, counter,
                                                    out_token, out_logprob);
    return acv_launch_status();
}

// ----------------------------------------------------------------------------- the k most probable tokens
// For each row the k largest logits in falling order (equal values: the lower index first) with their log
// probabilities logit - logsumexp(row), the normalisation of the chosen token's log probability
// (acvram/engine/sampler.py:103-117).  One block per row: a pass for the maximum and the sum of exponentials,
// then k passes, each finding the largest entry that comes after the one found before it.
#define TOPLP_MAX_K 64
__global__ void __launch_bounds__(SMP_THREADS)
top_logprobs_kernel(const float* __restrict__ logits, int ld, int V, int k, int* __restrict__ out_ids,
                    float* __restrict__ out_lp) {
    __shared__ float redf[32];
    __shared__ int redi[32];
    const float* row = logits + (size_t)blockIdx.x * ld;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, row[i]);
    mx = block_reduce_max(mx, redf);
    float sum = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) sum += __expf(row[i] - mx);
    sum = block_reduce_sum(sum, redf);
    const float lse = mx + logf(sum);
    float prev_v = INFINITY;
    int prev_i = -1;
    for (int n = 0; n < k; ++n) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            const bool after = v < prev_v || (v == prev_v && i > prev_i);      // not yet given out
            if (after && v > -INFINITY && (v > best || (v == best && i < bi))) { best = v; bi = i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
        __syncthreads();
        if (lane == 0) { redf[warp] = best; redi[warp] = bi; }
        __syncthreads();
        best = lane < nwarp ? redf[lane] : -INFINITY;
        bi = lane < nwarp ? redi[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) {              // fewer than k finite entries are left (k > V, or a row of -inf)
            if (threadIdx.x == 0) { out_ids[(size_t)blockIdx.x * k + n] = -1; out_lp[(size_t)blockIdx.x * k + n] = -INFINITY; }
            continue;
        }
        if (threadIdx.x == 0) {
            out_ids[(size_t)blockIdx.x * k + n] = bi;
            out_lp[(size_t)blockIdx.x * k + n] = best - lse;
        }
        prev_v = best;
        prev_i = bi;
    }
}

// logits float [rows, V] (row stride ld); out_ids int [rows, k], out_lp float [rows, k]; 1 <= k <= 64.
ACV_API int acv_top_logprobs(const float* logits, int ld, int rows, int V, int k, int* out_ids, float* out_lp,
                             cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (V <= 0 || k < 1 || k > TOPLP_MAX_K) return ACV_ERR_SIZE;
    top_logprobs_kernel<<<rows, SMP_THREADS, 0, stream>>>(logits, ld, V, k, out_ids, out_lp);
    return acv_launch_status();
}

ACV_TL_EXPORT(sampling)
