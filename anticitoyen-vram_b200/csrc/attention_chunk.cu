// Paged causal flash attention for portions of prompts (two or more query tokens
// of one request in a step), bfloat16.
//
// One CTA per (tile of 128 query tokens of one request, query head); its eight
// warps take 16 query rows each.  It serves the shapes the tcgen05 kernel (attention_tc.cu) does not take.  Keys and values come from the request's pages,
// earlier portions and this step's own tokens alike (they were appended before),
// in tiles of 64 keys, two in flight.  The query at absolute position p sees the
// keys j <= p, and with a window w > 0 only j > p - w: the mask follows absolute
// positions, so a portion that starts anywhere in the prompt is right
// (acvram/engine/layers.py:1020-1041).  The reference runs this case as a Python
// loop over requests that gathers the cached prefix into a dense copy and calls
// SDPA (acvram/engine/attention.py:519-584).
// QK^T and PV run on mma.sync m16n8k16 with float accumulation; the running
// maximum and sum of the softmax are float.
#include "mma_tiles.cuh"

#define AC_THREADS 256
#define AC_BM 128
#define AC_BN 64
#define AC_LOG2E 1.4426950408889634f

template <int D>
__global__ void __launch_bounds__(AC_THREADS)
attn_chunk_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                  const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages, const int* __restrict__ tile_seq,
                  const int* __restrict__ tile_q0, const int* __restrict__ cu_q, const int* __restrict__ kv_len,
                  const int* __restrict__ block_table, int bt_stride, const int* __restrict__ bt_rows, int NH, int NKV, int page_size, int page_shift,
                  int pg_cap, int num_pages, float scale, int window) {
    constexpr int CH = D / 8;
    constexpr int TILE_BYTES = AC_BN * D * 2;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* q_s = smem;                       // [128][D]
    unsigned char* k_s = smem + AC_BM * D * 2;       // [2][64][D]
    unsigned char* v_s = k_s + 2 * TILE_BYTES;       // [2][64][D]
    int* pg_s = reinterpret_cast<int*>(v_s + 2 * TILE_BYTES);   // [pg_cap] pages of the keys this tile reads

    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int seq = tile_seq[blockIdx.x], q0 = tile_q0[blockIdx.x];
    const int h = blockIdx.y;
    const int kvh = h / (NH / NKV);
    const int tok0 = cu_q[seq] + q0;
    const int q_len = cu_q[seq + 1] - cu_q[seq];
    const int rows = min(AC_BM, q_len - q0);
    const int pos0 = kv_len[seq] - q_len + q0;          // absolute position of the tile's first query
    const int* bt = block_table + (size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride;
    const int hi = pos0 + rows - 1;                     // last key any row of the tile sees
    const int lo = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int j_first = lo & ~(AC_BN - 1);
    const int n_tiles = (hi - j_first) / AC_BN + 1;

    for (int id = tid; id < AC_BM * CH; id += AC_THREADS) {
        const int r = id / CH, c = id % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < rows) v = *reinterpret_cast<const uint4*>(q + (size_t)(tok0 + r) * q_stride + (size_t)h * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = v;
    }

    // the block-table entries of the keys this tile reads, looked up once
    const int first_pg = page_shift >= 0 ? j_first >> page_shift : j_first / page_size;
    const int n_pg = (page_shift >= 0 ? hi >> page_shift : hi / page_size) - first_pg + 1;
    const bool pg_cached = n_pg <= pg_cap;
    if (pg_cached)
        for (int i = tid; i < n_pg; i += AC_THREADS) pg_s[i] = bt[first_pg + i];
    __syncthreads();

    // With pages of 16 keys or a multiple, each run of 16 rows of a tile lies in one page and is one
    // contiguous run of 16*D elements: one table lookup per 16 rows, fixed offsets for every thread.
    const bool contiguous = page_shift >= 4 && pg_cached;
    constexpr int ROWS_PER_IT = AC_THREADS / CH;          // rows the CTA covers with one copy instruction
    const int t_row = tid / CH, t_c = tid % CH;

    auto load_tile = [&](int t, int stage) {
        const int j0 = j_first + t * AC_BN;
        if (contiguous) {
#pragma unroll
            for (int it = 0; it < AC_BN / ROWS_PER_IT; ++it) {
                const int r = t_row + it * ROWS_PER_IT;
                const int j = j0 + r;
                bool ok = j <= hi && j >= lo;
                size_t row_off = 0;
                if (ok) {
                    const int pg = pg_s[(j >> page_shift) - first_pg];
                    ok = pg >= 0 && pg < num_pages;
                    row_off = (((size_t)pg * NKV + kvh) * page_size + (j & (page_size - 1))) * D + t_c * 8;
                }
                const int off = stage * TILE_BYTES + tile_off<D>(r, t_c);
                cp_async16(smem_u32(k_s + off), ok ? (const void*)(k_pages + row_off) : (const void*)k_pages, ok);
                cp_async16(smem_u32(v_s + off), ok ? (const void*)(v_pages + row_off) : (const void*)v_pages, ok);
            }
            return;
        }
        for (int id = tid; id < AC_BN * CH; id += AC_THREADS) {
            const int r = id / CH, c = id % CH;
            const int j = j0 + r;
            bool ok = j <= hi && j >= lo;
            size_t row_off = 0;
            if (ok) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / page_size;
                const int in_pg = page_shift >= 0 ? j & (page_size - 1) : j - pi * page_size;
                const int pg = pg_cached ? pg_s[pi - first_pg] : bt[pi];
                ok = pg >= 0 && pg < num_pages;
                row_off = (((size_t)pg * NKV + kvh) * page_size + in_pg) * D + c * 8;
            }
            const int off = stage * TILE_BYTES + tile_off<D>(r, c);
            cp_async16(smem_u32(k_s + off), ok ? (const void*)(k_pages + row_off) : (const void*)k_pages, ok);
            cp_async16(smem_u32(v_s + off), ok ? (const void*)(v_pages + row_off) : (const void*)v_pages, ok);
        }
    };

    load_tile(0, 0);
    cp_async_commit();
    __syncthreads();

    const int mi = lane >> 3, lr = lane & 7;
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int kd = 0; kd < D / 16; ++kd)
        ldmatrix_x4(qf[kd], smem_u32(q_s + tile_off<D>(warp * 16 + (mi & 1) * 8 + lr, kd * 2 + (mi >> 1))));

    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale_log2 = scale * AC_LOG2E;
    // absolute positions of this thread's two rows
    const int p_row[2] = {pos0 + warp * 16 + (lane >> 2), pos0 + warp * 16 + (lane >> 2) + 8};

    for (int t = 0; t < n_tiles; ++t) {
        const int stage = t & 1;
        if (t + 1 < n_tiles) load_tile(t + 1, stage ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint32_t kb = smem_u32(k_s + stage * TILE_BYTES), vb = smem_u32(v_s + stage * TILE_BYTES);
        const int j0 = j_first + t * AC_BN;
        // a warp whose rows all come before this tile's first key has nothing to do in it
        const bool active = j0 <= pos0 + warp * 16 + 15 && warp * 16 < rows &&
                            (window <= 0 || j0 + AC_BN - 1 > pos0 + warp * 16 - window);
        if (active) {
            float s[AC_BN / 8][4];
#pragma unroll
            for (int nt = 0; nt < AC_BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[nt][e] = 0.f;
#pragma unroll
            for (int kd = 0; kd < D / 16; ++kd) {
#pragma unroll
                for (int np = 0; np < AC_BN / 16; ++np) {
                    uint32_t b[4];
                    ldmatrix_x4(b, kb + tile_off<D>(np * 16 + (mi >> 1) * 8 + lr, kd * 2 + (mi & 1)));
                    mma_bf16(s[2 * np], qf[kd], b[0], b[1]);
                    mma_bf16(s[2 * np + 1], qf[kd], b[2], b[3]);
                }
            }
            // Only tiles that cross a row's causal edge (or the window's lower edge) need the mask; the
            // scores stay unscaled: scale*log2(e) goes into the exponent's fused multiply-add.
            const bool need_mask = !(j0 + AC_BN - 1 <= pos0 + warp * 16 &&
                                     (window <= 0 || j0 > pos0 + warp * 16 + 15 - window));
            float mx[2] = {-INFINITY, -INFINITY};
            if (need_mask) {
#pragma unroll
                for (int nt = 0; nt < AC_BN / 8; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = j0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        const int p = p_row[e >> 1];
                        const bool seen = j <= p && (window <= 0 || j > p - window);
                        if (!seen) s[nt][e] = -INFINITY;
                    }
            }
#pragma unroll
            for (int nt = 0; nt < AC_BN / 8; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) mx[e >> 1] = fmaxf(mx[e >> 1], s[nt][e]);
            float alpha[2], m_use[2];
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
                mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
                const float m_new = fmaxf(m_run[hh], mx[hh] * scale_log2);
                m_use[hh] = m_new == -INFINITY ? 0.f : m_new;
                alpha[hh] = fast_exp2(m_run[hh] - m_use[hh]);
                m_run[hh] = m_new;
                l_run[hh] *= alpha[hh];
            }
            if (alpha[0] != 1.f || alpha[1] != 1.f) {       // the running maximum moved
#pragma unroll
                for (int i = 0; i < D / 8; ++i) {
                    acc[i][0] *= alpha[0]; acc[i][1] *= alpha[0];
                    acc[i][2] *= alpha[1]; acc[i][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int kp = 0; kp < AC_BN / 16; ++kp) {
                uint32_t pa[4];
                float pv[2][4];
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        pv[nt][e] = fast_exp2(fmaf(s[2 * kp + nt][e], scale_log2, -m_use[e >> 1]));
                        l_run[e >> 1] += pv[nt][e];
                    }
                pa[0] = pack_bf16(pv[0][0], pv[0][1]);
                pa[1] = pack_bf16(pv[0][2], pv[0][3]);
                pa[2] = pack_bf16(pv[1][0], pv[1][1]);
                pa[3] = pack_bf16(pv[1][2], pv[1][3]);
#pragma unroll
                for (int nd = 0; nd < D / 16; ++nd) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vb + tile_off<D>(kp * 16 + (mi & 1) * 8 + lr, nd * 2 + (mi >> 1)));
                    mma_bf16(acc[2 * nd], pa, b[0], b[1]);
                    mma_bf16(acc[2 * nd + 1], pa, b[2], b[3]);
                }
            }
        }
        __syncthreads();
    }
    cp_async_wait<0>();

#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
        l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
    }
    const int r0 = warp * 16 + (lane >> 2);
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
        const int r = r0 + hh * 8;
        if (r >= rows) continue;
        const float inv = l_run[hh] > 0.f ? 1.f / l_run[hh] : 0.f;
        bf16* o = out + (size_t)(tok0 + r) * out_stride + (size_t)h * D + (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            const __nv_bfloat162 v = __floats2bfloat162_rn(acc[i][2 * hh] * inv, acc[i][2 * hh + 1] * inv);
            *reinterpret_cast<__nv_bfloat162*>(o + i * 8) = v;
        }
    }
}

template <int D>
static int launch_chunk(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                        const void* v_pages, const int* tile_seq, const int* tile_q0, int n_tiles, const int* cu_q,
                        const int* kv_len, const int* block_table, int bt_stride, const int* bt_rows, int NH, int NKV, int page_size,
                        int num_pages, float scale, int window, int max_kv, cudaStream_t stream) {
    int page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if ((1 << b) == page_size) page_shift = b;
    int pg_cap = max_kv / page_size + 2;
    if (pg_cap > 16384) pg_cap = 16384;
    const int smem = AC_BM * D * 2 + 4 * AC_BN * D * 2 + pg_cap * 4;
    static AcvSmemConfig smem_config;          // per kernel instance and device
    if (int rc = acv_ensure_smem(smem_config, attn_chunk_kernel<D>, smem)) return rc;
    dim3 grid(n_tiles, NH);
    acv_launch(PDL_MISC, attn_chunk_kernel<D>, grid, AC_THREADS, smem, stream,
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages, tile_seq,
        tile_q0, cu_q, kv_len, block_table, bt_stride, bt_rows, NH, NKV, page_size, page_shift, pg_cap, num_pages, scale, window);
    return acv_launch_status();
}

// tile_seq / tile_q0: for each tile of 128 query tokens, its request's index in the batch and the offset of
// the tile's first token among the request's tokens of this step.
ACV_API int acv_attention_chunk(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                const void* v_pages, const int* tile_seq, const int* tile_q0, int n_tiles,
                                const int* cu_q, const int* kv_len, const int* block_table, int bt_stride, const int* bt_rows, int NH,
                                int NKV, int D, int page_size, int num_pages, float scale, int window, int max_kv,
                                cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (NKV <= 0 || NH % NKV || NH > 65535) return ACV_ERR_SIZE;
    if (((uintptr_t)q & 15) || ((size_t)q_stride * 2) % 16 || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
        ((uintptr_t)out & 3) || (out_stride & 1))
        return ACV_ERR_ALIGN;
#define AC_ARGS q, q_stride, out, out_stride, k_pages, v_pages, tile_seq, tile_q0, n_tiles, cu_q, kv_len, block_table, \
                bt_stride, bt_rows, NH, NKV, page_size, num_pages, scale, window, max_kv, stream
    switch (D) {
        case 64: return launch_chunk<64>(AC_ARGS);
        case 128: return launch_chunk<128>(AC_ARGS);
        default: return ACV_ERR_SIZE;
    }
#undef AC_ARGS
}
