// What the tensor-core products share: the parameters of one product and the epilogues that work on a tile whose
// lanes are output features (weights on the tensor core's M side, the form that steps of few tokens use): SiLU(gate)*up
// on pairs of features, the tile staged in shared memory as C has it and written in 16-byte rows, and the stacked
// q,k,v projection's own epilogue (per-head norm, rotation, append to the pages).
#pragma once

#include "tc_ptx.cuh"

#define GT_BM 128            // rows of the A operand per tile = UMMA M
#define GT_BK 64             // K elements per stage = one 128-byte swizzle row

struct GemmParams {
    int RA, RB, K;          // rows of the A operand, rows of the B operand, reduction length
    int M, N;               // output is C[M, N]
    int ldc;
    int swap;               // 0: A = x (rows = tokens), 1: A = weight (rows = features)
    int out_f32;
    int act;                // 1: output features come in (gate, up) pairs and C[:, n/2] = silu(gate) * up
    int tiles_a, tiles_b, splits, kb_per_split, n_kb;
    int group_a;            // rows of tiles that are walked together (see gt_tile_of)
    int early_w;            // 1: the weights were written long before this launch: their first tiles are loaded before the predecessor ends
    int cluster;            // 1: the splits of a tile are the CTAs of one cluster and are summed through its shared memory
    int stages;             // pipeline depth (2..8); shared memory = stages * (128 + BN) * 128 bytes
    int staged;             // 1: swapped roles, one work item per CTA, C aligned: the tile goes out through shared memory in 16-byte rows
    // stacked q,k,v projection (staged tiles, up to 32 tokens): per-head RMS norm of q and k, rotation, and the
    // append of k and v to their pages, made on the tile as it leaves; only the q columns of C are written
    int qkv;
    int q_heads, kv_heads, head_dim;            // head_dim 64 or 128
    const float* q_w;
    const float* k_w;
    float qk_eps;
    const float* cos_sin;                       // [table_rows][head_dim]: cos then sin, or null
    int table_rows;
    const int* positions;
    const int* seq_of_token;
    const int* block_table;
    int bt_stride;
    const int* bt_rows;                         // the row of block_table of each request of the batch (null: its index)
    bf16* k_pages;
    bf16* v_pages;
    int page_size, num_pages;
    void* C;
    float* workspace;       // [tiles][splits][BN][128] floats when splits > 1
    int* counters;          // [tiles], zero before and after
    int* status;            // 0, or the code of the wait that ran out
    // for the test of the bounded waits only (acv_gemm_tc_test_fault): polls before a wait gives up, and a k-block
    // whose loads the producer leaves out, so that the wait for it must run out (-1: none)
    unsigned int wait_limit;
    int skip_kb;
};

// SiLU(gate) * up with the roundings of the unfused path: the product's outputs are rounded to
// bfloat16, SiLU is computed in float and rounded, then the product is rounded.
__device__ __forceinline__ bf16 swiglu_pair(float gate, float up) {
    const float g = __bfloat162float(__float2bfloat16_rn(gate));
    const float u = __bfloat162float(__float2bfloat16_rn(up));
    const float s = __bfloat162float(__float2bfloat16_rn(silu_f32<bf16>(g)));
    return __float2bfloat16_rn(s * u);
}

// Swapped roles: features lie on lanes, an even lane holds the gate of 16 tokens and the next lane their up.  The two
// share the work: each sends the other the eight values that it does not need, the even lane makes the tokens 0..7,
// the odd lane the tokens 8..15 (all exchanges first, then the arithmetic, so that the eight chains run side by
// side: done token by token, with the odd lane idle, this took 75 ns a token).  Returns the first of this lane's tokens.
__device__ __forceinline__ int swiglu_lane_pair(const float (&v)[16], int lane, bf16 (&o)[8]) {
    const bool odd = lane & 1;
    float other[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) other[c] = __shfl_xor_sync(0xffffffffu, odd ? v[c] : v[c + 8], 1);
#pragma unroll
    for (int c = 0; c < 8; ++c) o[c] = swiglu_pair(odd ? other[c] : v[c], odd ? v[c + 8] : other[c]);
    return odd ? 8 : 0;
}

// Write 16 accumulator columns of one tensor-memory lane: row_a is the A-operand row the lane holds,
// col0 the B-operand row of v[0].  Executed by whole warps (the paired form shuffles between lanes).
__device__ __forceinline__ void gt_store16(const GemmParams& p, int row_a, int col0, const float (&v)[16], int lane) {
    if (p.act) {
        if (p.swap) {       // features lie on lanes: an even lane holds a gate, the next lane its up
            bf16 o[8];
            const int first = swiglu_lane_pair(v, lane, o);
            const int f = row_a & ~1;           // the pair's gate row
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const int m = col0 + first + c;
                if (f + 1 < p.N && m < p.M) ((bf16*)p.C)[(size_t)m * p.ldc + (f >> 1)] = o[c];
            }
        } else if (row_a < p.M) {   // features lie on columns: (v[0], v[1]), (v[2], v[3]) ...
            bf16* dst = (bf16*)p.C + (size_t)row_a * p.ldc + (col0 >> 1);
            bf16 o[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) o[k] = swiglu_pair(v[2 * k], v[2 * k + 1]);
            if (col0 + 16 <= p.N && (((uintptr_t)dst) & 15) == 0) {
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(o);
            } else {
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    if (col0 + 2 * k + 1 < p.N) dst[k] = o[k];
            }
        }
        return;
    }
    if (p.swap) {
        // C[token = col0 + c][feature = row_a]: lanes write neighbouring features
        if (row_a < p.N) {
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                const int m = col0 + c;
                if (m < p.M) {
                    if (p.out_f32) ((float*)p.C)[(size_t)m * p.ldc + row_a] = v[c];
                    else ((bf16*)p.C)[(size_t)m * p.ldc + row_a] = __float2bfloat16_rn(v[c]);
                }
            }
        }
    } else if (row_a < p.M) {
        if (p.out_f32) {
            float* dst = (float*)p.C + (size_t)row_a * p.ldc + col0;
#pragma unroll
            for (int c = 0; c < 16; ++c)
                if (col0 + c < p.N) dst[c] = v[c];
        } else {
            bf16* dst = (bf16*)p.C + (size_t)row_a * p.ldc + col0;
            if (col0 + 16 <= p.N && (((uintptr_t)dst) & 15) == 0) {
                __nv_bfloat162 o[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) o[k] = __floats2bfloat162_rn(v[2 * k], v[2 * k + 1]);
                ((uint4*)dst)[0] = reinterpret_cast<const uint4*>(o)[0];
                ((uint4*)dst)[1] = reinterpret_cast<const uint4*>(o)[1];
            } else {
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    if (col0 + c < p.N) dst[c] = __float2bfloat16_rn(v[c]);
            }
        }
    }
}

// Swapped roles put features on tensor-memory lanes and tokens on columns, the transpose of C's rows.
// With one work item per CTA the pipeline's shared memory is free once the accumulator is complete:
// the tile is put there as C has it ([token][feature of the tile], in the output type) and leaves in
// 16-byte pieces of whole rows, instead of one 2-byte store per token and thread.
// gt_stage16: 16 tokens (col0 ..) of the feature this lane holds (f = 0..127 within the tile).
__device__ __forceinline__ void gt_stage16(const GemmParams& p, unsigned char* stage, int f, int col0, const float (&v)[16], int lane) {
    if (p.act) {            // an even lane holds a gate, the next lane its up: 64 output features per tile
        bf16 o[8];
        const int first = swiglu_lane_pair(v, lane, o);
#pragma unroll
        for (int c = 0; c < 8; ++c) reinterpret_cast<bf16*>(stage)[(col0 + first + c) * 64 + (f >> 1)] = o[c];
    } else if (p.out_f32) {
#pragma unroll
        for (int c = 0; c < 16; ++c) reinterpret_cast<float*>(stage)[(col0 + c) * 128 + f] = v[c];
    } else {
#pragma unroll
        for (int c = 0; c < 16; ++c) reinterpret_cast<bf16*>(stage)[(col0 + c) * 128 + f] = __float2bfloat16_rn(v[c]);
    }
}
// gt_flush: the staged tile (tokens tb*BN .., features ta*128 ..) to C, by the 128 epilogue threads
__device__ __forceinline__ void gt_flush(const GemmParams& p, const unsigned char* stage, int ta, int tb, int bn, int et) {
    const int esz = p.out_f32 ? 4 : 2;
    const int feats = p.act ? 64 : 128;                    // output features of the tile
    const int n_out = p.act ? p.N >> 1 : p.N;
    const int f0 = ta * feats;
    const int row_bytes = feats * esz, chunks = row_bytes >> 4, per_chunk = 16 / esz;
    const int rows = min(bn, p.M - tb * bn);
    for (int q = et; q < rows * chunks; q += 128) {
        const int r = q / chunks, ch = q - r * chunks;
        const int f = f0 + ch * per_chunk;
        if (f >= n_out) continue;
        unsigned char* dst = (unsigned char*)p.C + ((size_t)(tb * bn + r) * p.ldc + f) * esz;
        const unsigned char* src = stage + r * row_bytes + (ch << 4);
        if (f + per_chunk <= n_out) {
            *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
        } else {
            for (int b = 0; b < (n_out - f) * esz; ++b) dst[b] = src[b];
        }
    }
}

// gt_flush_qkv: the staged tile of a stacked q,k,v projection.  A row of the tile is 128 features of one token:
// one head of 128 or two of 64.  The 16 threads of a row hold 8 features each; a head's threads add their squares
// for the RMS norm, and the rotation's partner (i +- D/2) sits half a head's threads away.  The arithmetic is the
// rotation kernel's (acvram/kernels/acvram_kernels.cu:4397-4430): norm, weight and rotation in float on the
// bfloat16 values of the projection, one rounding at the end.  aux: positions [BN], pages [BN], cos/sin rows [BN][D].
__device__ __forceinline__ void gt_flush_qkv(const GemmParams& p, const unsigned char* stage, const unsigned char* aux,
                                             int ta, int tb, int bn, int et) {
    const int D = p.head_dim, tph = D >> 3;                 // threads per head: 16 or 8
    const int* pos_s = reinterpret_cast<const int*>(aux);
    const int* pg_s = pos_s + bn;
    const float* cs_s = reinterpret_cast<const float*>(pg_s + bn);
    const int rows = min(bn, p.M - tb * bn);
    const int ch = et & 15;
    const int f = ta * 128 + ch * 8;                        // first of this thread's features in the stacked output
    const int head = f / D, off = f - head * D;             // the same in every turn of the loop
    const bool in_n = f < p.N;
    const bool is_q = head < p.q_heads, is_k = !is_q && head < p.q_heads + p.kv_heads, is_v = !is_q && !is_k;
    const float* w = is_q ? p.q_w : (is_k ? p.k_w : nullptr);
    float wv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) wv[e] = (w && in_n) ? w[off + e] : 1.f;
    const int i0 = off & ((D >> 1) - 1);                    // index of the first angle
    const bool first_half = off < (D >> 1);
    // a turn is eight rows; every thread takes every turn that has a token (the shuffles need all lanes), none takes the
    // turns beyond the tokens: with 8 requests in a tile of 16 that is one turn of this chain of shuffles instead of two
    for (int q = et; q < ((rows * 16 + 127) & ~127); q += 128) {
        const int r = q >> 4;
        const bool live = r < rows && in_n;
        float a[8];
        {
            uint4 raw = make_uint4(0, 0, 0, 0);
            if (r < bn) raw = *reinterpret_cast<const uint4*>(stage + r * 256 + (ch << 4));
            const bf16* e8 = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = __bfloat162float(e8[e]);
        }
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) ss += a[e] * a[e];
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        ss += __shfl_xor_sync(0xffffffffu, ss, 4);
        if (tph == 16) ss += __shfl_xor_sync(0xffffffffu, ss, 8);
        if (w) {
            const float inv = rsqrtf(ss / (float)D + p.qk_eps);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = a[e] * inv * wv[e];
        }
        const int pos = r < bn ? pos_s[r] : 0;
        float o[8];
        if (p.cos_sin) {
            const bool rotate = !is_v && pos >= 0 && pos < p.table_rows;
            const float* cs = cs_s + (size_t)(r < bn ? r : 0) * D;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float partner = __shfl_xor_sync(0xffffffffu, a[e], tph >> 1);
                const float c = cs[i0 + e], sn = cs[(D >> 1) + i0 + e];
                const float rot = first_half ? a[e] * c - partner * sn : a[e] * c + partner * sn;
                o[e] = rotate ? rot : a[e];
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = a[e];
        }
        if (!live) continue;
        bf16* dst = nullptr;
        if (is_q) {
            dst = (bf16*)p.C + (size_t)(tb * bn + r) * p.ldc + f;
        } else {
            const int pg = pg_s[r];
            if (pg >= 0) {
                const int kvh = is_k ? head - p.q_heads : head - p.q_heads - p.kv_heads;
                dst = (is_k ? p.k_pages : p.v_pages) +
                      (((size_t)pg * p.kv_heads + kvh) * p.page_size + (pos % p.page_size)) * D + off;
            }
        }
        if (dst) {
            uint4 out;
            out.x = pack2(__float_as_uint(o[0]), __float_as_uint(o[1]));
            out.y = pack2(__float_as_uint(o[2]), __float_as_uint(o[3]));
            out.z = pack2(__float_as_uint(o[4]), __float_as_uint(o[5]));
            out.w = pack2(__float_as_uint(o[6]), __float_as_uint(o[7]));
            *reinterpret_cast<uint4*>(dst) = out;
        }
    }
}

