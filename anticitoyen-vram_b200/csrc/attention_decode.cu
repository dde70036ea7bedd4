// Split-KV paged decode attention, bfloat16, grouped by kv-head.
//
// One CTA per (decoding request, kv-head, split of the context).  All query heads
// that share the kv-head (NH/NKV of them, at most 16) form the 16 rows of one
// tensor-core tile, so each key and value is read from memory once for the whole
// group.  The reference has such a kernel for int8 pages only and, for bf16
// pages, gathers the whole context into a dense copy before calling SDPA
// (acvram/engine/attention.py:651-654, acvram/memory/kvcache.py:735-768); its int8
// kernels have the same shape of work: partial (m, l, acc) per chunk, then a merge
// (acvram/kernels/acvram_kernels.cu:955-1361), and its Triton form lets the block
// that arrives last do the merge (acvram/kernels/attn_paginee.py:176-259), which
// is what happens here: no block ever waits for another.
//
// Keys and values stream through shared memory with 16-byte asynchronous copies.
// Each of the four warps takes every fourth tile of 16 keys of the CTA's range
// through a ring of buffers of its own (QK^T and PV on mma.sync m16n8k16, softmax
// state in float), so that several tiles are in flight for every warp and no warp
// waits for another; the warps merge at the end.  Rows of a tile are addressed
// through the block table one by one, so any page size works.
#include "mma_tiles.cuh"

#define AD_EARLY_KEYS 0
#define AD_TILE 64          // split boundaries fall on multiples of this many keys
#define AD_STAGES 3         // buffers in each warp's ring (2 and 4 measured slower on a B200)
#define AD_WARPS 4          // warps of a CTA where two CTAs share an SM
#define AD_WARPS_ALONE 8    // where a CTA has its SM to itself (a grid of no more CTAs than SMs)
#define AD_LOG2E 1.4426950408889634f

template <int D, int NW>
__global__ void __launch_bounds__(NW * 32)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                   const bf16* __restrict__ k_pages, const bf16* __restrict__ v_pages,
                   const int* __restrict__ dec_tokens, const int* __restrict__ dec_seqs,
                   const int* __restrict__ kv_len, const int* __restrict__ block_table, int bt_stride,
                   const int* __restrict__ bt_rows, int NH, int NKV, int page_size, int page_shift, int pg_cap, int num_pages, float scale, int window, int n_splits,
                   float* __restrict__ part_acc, float* __restrict__ part_ml, int* __restrict__ counters,
                   int cluster_merge) {
    constexpr int CH = D / 8;                 // 16-byte chunks per row
    constexpr int AD_THREADS = NW * 32;
    constexpr int WT_BYTES = 16 * D * 2;                         // 16 keys (or values) of one kv-head
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* ring = smem;                                  // [NW warps][AD_STAGES][K, V][16][D]
    int* pg_s = reinterpret_cast<int*>(ring + NW * AD_STAGES * 2 * WT_BYTES);   // [pg_cap] pages of this CTA's keys
    unsigned char* q_s = reinterpret_cast<unsigned char*>(pg_s + ((pg_cap + 31) & ~31));   // [16][D], until they are in registers
    // cluster merge, in rank 0: the partial results of the splits 1.. as [n_splits - 1][NH/NKV][D + 2], over the queries
    // (the peers write here at their end, and no sooner than every thread of rank 0 has its queries in registers)
    float* cm_s = reinterpret_cast<float*>(q_s);
    __shared__ int is_last_s;

    ACV_TL(TL_ATTN_DECODE, 0);
    pdl_launch_dependents();
    // What follows up to pdl_wait reads only what was written before this step's first kernel began (the step's index
    // arrays, the block table, keys and values of earlier steps): it runs while the projection before this kernel still
    // does.  The step's own query and its newest key and value are that projection's output and wait for it.
    const bool in_cluster = cluster_merge && n_splits > 1;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int item = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int tok = dec_tokens[item], seq = dec_seqs[item];
    const int n_rep = NH / NKV;
    const int* bt = block_table + (size_t)(bt_rows ? bt_rows[seq] : seq) * bt_stride;   // the request's row of the table
    const int p = kv_len[seq] - 1;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    const int n_keys = p + 1 - lo;
    const int chunk = (((n_keys + n_splits - 1) / n_splits) + AD_TILE - 1) & ~(AD_TILE - 1);
    const int beg = lo + split * chunk;
    const int end = min(beg + chunk, p + 1);
    const int n_tiles = beg < end ? (end - beg + AD_TILE - 1) / AD_TILE : 0;   // > 0: this split has keys

    // the block-table entries of this CTA's keys, read once (a tile's copies then wait for no lookup)
    const int first_pg = page_shift >= 0 ? beg >> page_shift : beg / page_size;
    const int n_pg = n_tiles > 0 ? (page_shift >= 0 ? (end - 1) >> page_shift : (end - 1) / page_size) - first_pg + 1 : 0;
    const bool pg_cached = n_pg <= pg_cap;
    if (pg_cached)
        for (int i = tid; i < n_pg; i += AD_THREADS) pg_s[i] = bt[first_pg + i];
    __syncthreads();

    // Each warp streams its own keys: the CTA's range is cut into tiles of 16 keys, warp w takes the
    // tiles w, w+NW, w+2NW ... through a ring of AD_STAGES buffers of its own, so that several tiles
    // are in flight for every warp and no warp waits for another inside the loop.
    const int n_wt = beg < end ? (end - beg + 15) / 16 : 0;
    const int my_n = n_wt > warp ? (n_wt - warp + NW - 1) / NW : 0;
    unsigned char* my_ring = ring + warp * (AD_STAGES * 2 * WT_BYTES);

    // With pages of 16 keys or a multiple, and a range that starts on a multiple of 16, a tile lies
    // in one page and its 16 rows are one contiguous run of 16*D elements: one table lookup per
    // tile, and every lane copies fixed offsets of that run.
    const bool contiguous = page_shift >= 4 && (beg & 15) == 0 && pg_cached;
    const int lane_row = lane / CH, lane_c = lane % CH;       // this lane's first row and its chunk in the row
    constexpr int ROWS_PER_IT = 32 / CH;                      // rows a warp covers with one copy instruction

    auto load_wt = [&](int i, int stage) {
        const int j0 = beg + (warp + NW * i) * 16;
        unsigned char* kdst = my_ring + stage * 2 * WT_BYTES;
        unsigned char* vdst = kdst + WT_BYTES;
        if (contiguous) {
            const int pg = pg_s[(j0 >> page_shift) - first_pg];
            const bool pg_ok = pg >= 0 && pg < num_pages;
            const size_t base = (((size_t)(pg_ok ? pg : 0) * NKV + kvh) * page_size + (j0 & (page_size - 1))) * D;
            const bf16* ksrc = k_pages + base + lane * 8;
            const bf16* vsrc = v_pages + base + lane * 8;
            const int rows_left = end - j0;                   // rows >= rows_left are beyond the range: zero
#pragma unroll
            for (int it = 0; it < 16 / ROWS_PER_IT; ++it) {
                const int r = lane_row + it * ROWS_PER_IT;
                const bool ok = pg_ok && r < rows_left;
                const int off = tile_off<D>(r, lane_c);
                cp_async16(smem_u32(kdst + off), ok ? (const void*)(ksrc + it * 256) : (const void*)k_pages, ok);
                cp_async16(smem_u32(vdst + off), ok ? (const void*)(vsrc + it * 256) : (const void*)v_pages, ok);
            }
            return;
        }
#pragma unroll
        for (int id = lane; id < 16 * CH; id += 32) {
            const int r = id / CH, c = id % CH;
            const int j = j0 + r;
            bool ok = j < end;
            size_t row_off = 0;
            if (ok) {
                const int pi = page_shift >= 0 ? j >> page_shift : j / page_size;
                const int in_pg = page_shift >= 0 ? j & (page_size - 1) : j - pi * page_size;
                const int pg = pg_cached ? pg_s[pi - first_pg] : bt[pi];
                ok = pg >= 0 && pg < num_pages;
                row_off = (((size_t)pg * NKV + kvh) * page_size + in_pg) * D + c * 8;
            }
            const int off = tile_off<D>(r, c);
            cp_async16(smem_u32(kdst + off), ok ? (const void*)(k_pages + row_off) : (const void*)k_pages, ok);
            cp_async16(smem_u32(vdst + off), ok ? (const void*)(v_pages + row_off) : (const void*)v_pages, ok);
        }
    };

    // The first tiles of the ring could go now as far as they hold keys of earlier steps only (the newest key, at p, is
    // written by the projection before this kernel).  Measured, that gains nothing: the projection is bound by memory
    // and the early copies take from it what they save here (3.799 against 3.789 ms a step); what pays is that the index
    // reads above, three dependent round trips, are over when the wait ends (3.739 ms).  AD_EARLY_KEYS keeps the form.
    int early = 0;
#pragma unroll
    for (int st = 0; st < AD_STAGES - 1; ++st) {
        if (AD_EARLY_KEYS && early == st && st < my_n && beg + (warp + NW * st) * 16 + 16 <= p) {
            load_wt(st, st);
            cp_async_commit();
            ++early;
        }
    }
    pdl_wait();
    // ---- queries of the group into shared memory (rows >= n_rep are zero)
    for (int id = tid; id < 16 * CH; id += AD_THREADS) {
        const int r = id / CH, c = id % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (r < n_rep) v = *reinterpret_cast<const uint4*>(q + (size_t)tok * q_stride + (size_t)(kvh * n_rep + r) * D + c * 8);
        *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = v;
    }
#pragma unroll
    for (int st = 0; st < AD_STAGES - 1; ++st) {
        if (st >= early) {
            if (st < my_n) load_wt(st, st);
            cp_async_commit();
        }
    }
    __syncthreads();            // the queries are in shared memory

    // ---- query fragments (A operand), kept in registers for the whole kernel
    uint32_t qf[D / 16][4];
    {
        const int mi = lane >> 3, r = lane & 7;
#pragma unroll
        for (int kd = 0; kd < D / 16; ++kd)
            ldmatrix_x4(qf[kd], smem_u32(q_s + tile_off<D>((mi & 1) * 8 + r, kd * 2 + (mi >> 1))));
    }
    // the splits of one cluster write their partial results into rank 0's shared memory at the end, where its queries
    // lay: a CTA may do so only when it knows that rank 0 has started and no longer reads them, which is what the first
    // phase of the cluster's barrier tells it.  Every thread arrives when its own reads have returned (the arrival takes
    // the loaded registers as operands); it publishes nothing, so it needs no release, which here would wait for the
    // copies of the first tiles that are under way (measured: half a microsecond a launch).
    if (in_cluster) {
        uint32_t seen = 0;
#pragma unroll
        for (int kd = 0; kd < D / 16; ++kd) seen |= qf[kd][0] | qf[kd][1] | qf[kd][2] | qf[kd][3];
        asm volatile("{\n.reg .pred p;\nsetp.eq.u32 p, %0, 0xffffffff;\nbarrier.cluster.arrive.relaxed.aligned;\n}" :: "r"(seen) : "memory");
    }

    float acc[D / 8][4];
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const float scale_log2 = scale * AD_LOG2E;
    const int mi = lane >> 3, lr = lane & 7;

    int stage = 0;
    for (int i = 0; i < my_n; ++i) {
        {
            const int nxt = i + AD_STAGES - 1;
            int nxt_stage = stage + AD_STAGES - 1;
            if (nxt_stage >= AD_STAGES) nxt_stage -= AD_STAGES;
            if (nxt < my_n) load_wt(nxt, nxt_stage);
            cp_async_commit();
        }
        cp_async_wait<AD_STAGES - 1>();
        __syncwarp();
        const uint32_t kb = smem_u32(my_ring + stage * 2 * WT_BYTES), vb = kb + WT_BYTES;
        const int jw = beg + (warp + NW * i) * 16;       // first key of this tile
        {
            float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
            for (int kd = 0; kd < D / 16; ++kd) {
                uint32_t b[4];
                ldmatrix_x4(b, kb + tile_off<D>((mi >> 1) * 8 + lr, kd * 2 + (mi & 1)));
                mma_bf16(s[0], qf[kd], b[0], b[1]);
                mma_bf16(s[1], qf[kd], b[2], b[3]);
            }
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = jw + nt * 8 + (lane & 3) * 2 + (e & 1);
                    const float v = j < end ? s[nt][e] * scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    mx[e >> 1] = fmaxf(mx[e >> 1], v);
                }
            float alpha[2], m_use[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
                mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
                const float m_new = fmaxf(m_run[h], mx[h]);
                m_use[h] = m_new == -INFINITY ? 0.f : m_new;
                alpha[h] = exp2f(m_run[h] - m_use[h]);
                m_run[h] = m_new;
                l_run[h] *= alpha[h];
            }
            uint32_t pa[4];
            float pv[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    pv[nt][e] = exp2f(s[nt][e] - m_use[e >> 1]);
                    l_run[e >> 1] += pv[nt][e];
                }
            pa[0] = pack_bf16(pv[0][0], pv[0][1]);
            pa[1] = pack_bf16(pv[0][2], pv[0][3]);
            pa[2] = pack_bf16(pv[1][0], pv[1][1]);
            pa[3] = pack_bf16(pv[1][2], pv[1][3]);
            if (alpha[0] != 1.f || alpha[1] != 1.f) {       // the running maximum moved: rescale what is summed so far
#pragma unroll
                for (int ii = 0; ii < D / 8; ++ii) {
                    acc[ii][0] *= alpha[0]; acc[ii][1] *= alpha[0];
                    acc[ii][2] *= alpha[1]; acc[ii][3] *= alpha[1];
                }
            }
#pragma unroll
            for (int nd = 0; nd < D / 16; ++nd) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vb + tile_off<D>((mi & 1) * 8 + lr, nd * 2 + (mi >> 1)));
                mma_bf16(acc[2 * nd], pa, b[0], b[1]);
                mma_bf16(acc[2 * nd + 1], pa, b[2], b[3]);
            }
        }
        __syncwarp();
        stage = stage + 1 == AD_STAGES ? 0 : stage + 1;
    }
    cp_async_wait<0>();
    __syncthreads();
    if (tid == 0) ACV_TL_MARK(TL_M_ATTN_LOOP_DONE);

    // ---- merge the four warps through shared memory (the tiles are no longer needed)
    float* wm = reinterpret_cast<float*>(ring);           // [NW][16]
    float* wl = wm + NW * 16;                             // [NW][16]
    float* wacc = wl + NW * 16;                           // [NW][16][D]
    float* own_s = wacc + NW * 16 * D;                    // [NH/NKV][D + 2]: rank 0's own partial result (cluster merge)
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
        l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
    }
    {
        const int r0 = lane >> 2, c0 = (lane & 3) * 2;
        if ((lane & 3) == 0) {
            wm[warp * 16 + r0] = m_run[0]; wm[warp * 16 + r0 + 8] = m_run[1];
            wl[warp * 16 + r0] = l_run[0]; wl[warp * 16 + r0 + 8] = l_run[1];
        }
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
            float* a0 = wacc + ((warp * 16 + r0) * D) + i * 8 + c0;
            float* a1 = wacc + ((warp * 16 + r0 + 8) * D) + i * 8 + c0;
            a0[0] = acc[i][0]; a0[1] = acc[i][1];
            a1[0] = acc[i][2]; a1[1] = acc[i][3];
        }
    }
    __syncthreads();

    const size_t part = ((size_t)item * NKV + kvh) * n_splits + split;
    if (in_cluster) cluster_wait();          // long passed: the peers arrived when they began
    for (int idx = tid; idx < n_rep * D; idx += AD_THREADS) {
        const int r = idx / D, d = idx % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; ++w) M = fmaxf(M, wm[w * 16 + r]);
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < NW; ++w) {
                const float f = exp2f(wm[w * 16 + r] - M);
                L += wl[w * 16 + r] * f;
                O += wacc[(w * 16 + r) * D + d] * f;
            }
        }
        if (n_splits == 1) {
            out[(size_t)tok * out_stride + (size_t)(kvh * n_rep + r) * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        } else if (cluster_merge) {
            // the splits of a (request, kv-head) are the CTAs of one cluster: each puts its partial into rank 0's
            // shared memory, rank 0 merges them after the cluster barrier
            if (split == 0) {
                float* dst = own_s + r * (D + 2);
                dst[d] = O;
                if (d == 0) {
                    dst[D] = M;
                    dst[D + 1] = L;
                }
            } else {
                const uint32_t dst = cluster_map(smem_u32(cm_s), 0) + (((split - 1) * n_rep + r) * (D + 2) + d) * 4;
                cluster_store_f32(dst, O);
                if (d == 0) {
                    cluster_store_f32(dst + D * 4, M);
                    cluster_store_f32(dst + (D + 1) * 4, L);
                }
            }
        } else {
            part_acc[(part * n_rep + r) * D + d] = O;
            if (d == 0) {
                part_ml[(part * n_rep + r) * 2] = M;
                part_ml[(part * n_rep + r) * 2 + 1] = L;
            }
        }
    }
    if (n_splits == 1) return;
    if (cluster_merge) {
        cluster_sync_all();
        if (split != 0) return;
        for (int idx = tid; idx < n_rep * D; idx += AD_THREADS) {
            const int r = idx / D, d = idx % D;
            float M = own_s[r * (D + 2) + D];
            for (int sp = 1; sp < n_splits; ++sp) M = fmaxf(M, cm_s[((sp - 1) * n_rep + r) * (D + 2) + D]);
            float L = 0.f, O = 0.f;
            if (M != -INFINITY) {
                for (int sp = 0; sp < n_splits; ++sp) {          // split order: the sum does not depend on timing
                    const float* ps = sp == 0 ? own_s + r * (D + 2) : cm_s + ((sp - 1) * n_rep + r) * (D + 2);
                    const float f = exp2f(ps[D] - M);
                    L += ps[D + 1] * f;
                    O += ps[d] * f;
                }
            }
            out[(size_t)tok * out_stride + (size_t)(kvh * n_rep + r) * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        }
        return;
    }

    // ---- the block that arrives last merges the splits, in split order
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const int old = atomicAdd(&counters[item * NKV + kvh], 1);
        is_last_s = old == n_splits - 1;
    }
    __syncthreads();
    if (!is_last_s) return;
    __threadfence();
    const size_t base = ((size_t)item * NKV + kvh) * n_splits;
    for (int idx = tid; idx < n_rep * D; idx += AD_THREADS) {
        const int r = idx / D, d = idx % D;
        // eight splits' loads are under way at a time (one after the other, every split would cost a round trip to the
        // L2 cache); the sums still run in split order
        const float2* ml = reinterpret_cast<const float2*>(part_ml) + base * n_rep + r;
        const float* pa = part_acc + (base * n_rep + r) * D + d;
        float M = -INFINITY;
        for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
            float m[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) m[u] = sp0 + u < n_splits ? __ldcg(&ml[(size_t)(sp0 + u) * n_rep]).x : -INFINITY;
#pragma unroll
            for (int u = 0; u < 8; ++u) M = fmaxf(M, m[u]);
        }
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
            for (int sp0 = 0; sp0 < n_splits; sp0 += 8) {
                float2 v[8];
                float o[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const bool ok = sp0 + u < n_splits;
                    v[u] = ok ? __ldcg(&ml[(size_t)(sp0 + u) * n_rep]) : make_float2(-INFINITY, 0.f);
                    o[u] = ok ? __ldcg(&pa[(size_t)(sp0 + u) * n_rep * D]) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    if (sp0 + u < n_splits) {
                        const float f = exp2f(v[u].x - M);
                        L += v[u].y * f;
                        O += o[u] * f;
                    }
                }
            }
        }
        out[(size_t)tok * out_stride + (size_t)(kvh * n_rep + r) * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
    if (tid == 0) counters[item * NKV + kvh] = 0;   // ready for the next launch
}

// Dynamic shared memory of a CTA: the four warps' rings, the block-table entries of its keys, and the queries or, with a
// merge inside the cluster and in their place, the partial results of the other splits (used in rank 0).
static int decode_smem_bytes(int D, int n_rep, int page_size, int window, int n_splits, int max_kv, int cluster_merge,
                             int warps, int* pg_cap_out) {
    const int keys = window > 0 && window < max_kv ? window : max_kv;
    const int chunk = (((keys + n_splits - 1) / n_splits) + AD_TILE - 1) & ~(AD_TILE - 1);
    int pg_cap = chunk / page_size + 2;
    if (pg_cap > 8192) pg_cap = 8192;
    *pg_cap_out = pg_cap;
    const int queries = 16 * D * 2;
    const int partials = cluster_merge ? (n_splits - 1) * n_rep * (D + 2) * 4 : 0;     // where the queries lay
    return warps * AD_STAGES * 2 * 16 * D * 2 + ((pg_cap + 31) & ~31) * 4 + (partials > queries ? partials : queries);
}

// One record per kernel instance of the shared memory it has been allowed so far: the launch and the residency question
// must not keep two, the second would lower what the first has raised.
template <int D, int NW>
static AcvSmemConfig& decode_smem_config() {
    static AcvSmemConfig config;
    return config;
}

template <int D, int NW>
static int decode_resident(int smem, int cluster) {
    if (int rc = acv_ensure_smem(decode_smem_config<D, NW>(), attn_decode_kernel<D, NW>, smem)) return rc > 0 ? ACV_ERR_SIZE : rc;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        cudaGetLastError();
        return ACV_ERR_SIZE;
    }
    if (cluster <= 1) {
        int per_sm = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_kernel<D, NW>, NW * 32, smem) != cudaSuccess) {
            cudaGetLastError();
            return ACV_ERR_SIZE;
        }
        return per_sm * sms;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, cluster);
    cfg.blockDim = dim3(NW * 32);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = cluster;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, attn_decode_kernel<D, NW>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return ACV_ERR_SIZE;
    }
    return clusters * cluster;
}

// A grid small enough to have an SM for every CTA gets one: with room for two, the CTAs of a cluster are put two to an
// SM, half the SMs stay empty and the step of a single request measured 1.9 % slower.  Such a grid runs the kernel with
// twice the warps and rings, whose shared memory leaves no room for a second CTA (and is raised to that size where a
// small head would).  Returns whether the grid is one: no more CTAs than the device holds one to an SM in clusters of this size
// (asked of the runtime once per device and cluster size).  ``alone`` receives the least size that keeps an SM for one CTA.
template <int D>
static bool decode_grid_has_sms(int cluster, long long ctas, int* alone) {
    static std::mutex mu;
    static int fit[64][9];          // [device][cluster size]: CTAs resident with one to an SM; -1 = cannot be had
    static int alone_bytes[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || cluster < 1 || cluster > 8) return false;
    std::lock_guard<std::mutex> lock(mu);
    if (!alone_bytes[dev]) {
        int per_sm = 0, reserved = 0, per_block = 0;
        if (cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&reserved, cudaDevAttrReservedSharedMemoryPerBlock, dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&per_block, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
            cudaGetLastError();
            alone_bytes[dev] = -1;
        } else {
            const int want = per_sm / 2 - reserved + 128;      // two of these and their reserves exceed an SM
            alone_bytes[dev] = want <= per_block ? want : -1;
        }
    }
    if (alone_bytes[dev] < 0) return false;
    *alone = alone_bytes[dev];
    if (!fit[dev][cluster]) {
        const int n = decode_resident<D, AD_WARPS_ALONE>(alone_bytes[dev], cluster);
        fit[dev][cluster] = n > 0 ? n : -1;
    }
    return ctas <= fit[dev][cluster];
}

template <int D, int NW>
static int launch_decode_with(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                              const void* v_pages, const int* dec_tokens, const int* dec_seqs, int n_dec, const int* kv_len,
                              const int* block_table, int bt_stride, const int* bt_rows, int NH, int NKV, int page_size,
                              int page_shift, int pg_cap, int num_pages, float scale, int window, int n_splits,
                              float* part_acc, float* part_ml, int* counters, int cluster_merge, int smem,
                              cudaStream_t stream) {
    if (int rc = acv_ensure_smem(decode_smem_config<D, NW>(), attn_decode_kernel<D, NW>, smem)) return rc;
    dim3 grid(n_dec, NKV, n_splits);
    acv_launch_cluster(PDL_ATTN, dim3(1, 1, cluster_merge ? n_splits : 1), attn_decode_kernel<D, NW>, grid, NW * 32, smem,
        stream, (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pages, (const bf16*)v_pages, dec_tokens,
        dec_seqs, kv_len, block_table, bt_stride, bt_rows, NH, NKV, page_size, page_shift, pg_cap, num_pages, scale, window,
        n_splits, part_acc, part_ml, counters, cluster_merge);
    return acv_launch_status();
}

template <int D>
static int launch_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                         const void* v_pages, const int* dec_tokens, const int* dec_seqs, int n_dec, const int* kv_len,
                         const int* block_table, int bt_stride, const int* bt_rows, int NH, int NKV, int page_size,
                         int num_pages, float scale, int window, int n_splits, float* part_acc, float* part_ml, int* counters,
                         int max_kv, int cluster_merge, cudaStream_t stream) {
    int page_shift = -1;
    for (int b = 0; b < 31; ++b)
        if ((1 << b) == page_size) page_shift = b;
    if (n_splits < 2 || n_splits > 8) cluster_merge = 0;
    int pg_cap = 0, alone = 0;
    const int cluster = cluster_merge ? n_splits : 1;
#define AD_LAUNCH_ARGS q, q_stride, out, out_stride, k_pages, v_pages, dec_tokens, dec_seqs, n_dec, kv_len, block_table, \
                       bt_stride, bt_rows, NH, NKV, page_size, page_shift, pg_cap, num_pages, scale, window, n_splits, \
                       part_acc, part_ml, counters, cluster_merge
    if (decode_grid_has_sms<D>(cluster, (long long)n_dec * NKV * n_splits, &alone)) {
        int smem = decode_smem_bytes(D, NH / NKV, page_size, window, n_splits, max_kv, cluster_merge, AD_WARPS_ALONE, &pg_cap);
        if (smem < alone) smem = alone;
        int dev = 0, per_block = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&per_block, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (smem <= per_block) return launch_decode_with<D, AD_WARPS_ALONE>(AD_LAUNCH_ARGS, smem, stream);
        // too many partial results beside eight rings: four warps, still one CTA to an SM
        smem = decode_smem_bytes(D, NH / NKV, page_size, window, n_splits, max_kv, cluster_merge, AD_WARPS, &pg_cap);
        return launch_decode_with<D, AD_WARPS>(AD_LAUNCH_ARGS, smem < alone ? alone : smem, stream);
    }
    const int smem = decode_smem_bytes(D, NH / NKV, page_size, window, n_splits, max_kv, cluster_merge, AD_WARPS, &pg_cap);
    return launch_decode_with<D, AD_WARPS>(AD_LAUNCH_ARGS, smem, stream);
#undef AD_LAUNCH_ARGS
}

// bt_rows (may be null): the row of block_table that belongs to each request of the batch (null: row = its index).
// Scratch, given by the caller: part_acc holds n_dec*NKV*n_splits*(NH/NKV)*D floats, part_ml
// n_dec*NKV*n_splits*(NH/NKV)*2 floats, counters n_dec*NKV ints that are zero before the first call
// (the kernel leaves them zero).  scratch_floats / scratch_counters say how much the caller gave.
ACV_API int acv_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                 const void* v_pages, const int* dec_tokens, const int* dec_seqs, int n_dec,
                                 const int* kv_len, const int* block_table, int bt_stride, const int* bt_rows, int NH,
                                 int NKV, int D, int page_size, int num_pages, float scale, int window, int n_splits, float* part_acc,
                                 float* part_ml, int* counters, long long scratch_floats, long long scratch_ml_floats,
                                 long long scratch_counters, int max_kv, int cluster_merge, cudaStream_t stream) {
    if (n_dec <= 0) return 0;
    if (NKV <= 0 || NH % NKV || NH / NKV > 16 || n_splits < 1 || n_splits > 65535 || NKV > 65535) return ACV_ERR_SIZE;
    if (((uintptr_t)q & 15) || ((size_t)q_stride * 2) % 16 || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15))
        return ACV_ERR_ALIGN;
    const long long n_rep = NH / NKV;
    if (n_splits > 1 && !(cluster_merge && n_splits <= 8)) {
        const long long parts = (long long)n_dec * NKV * n_splits;
        if (parts * n_rep * D > scratch_floats || parts * n_rep * 2 > scratch_ml_floats ||
            (long long)n_dec * NKV > scratch_counters)
            return ACV_ERR_SCRATCH;
        if ((uintptr_t)part_ml & 7) return ACV_ERR_ALIGN;      // (max, sum) are read as pairs
    }
#define AD_ARGS q, q_stride, out, out_stride, k_pages, v_pages, dec_tokens, dec_seqs, n_dec, kv_len, block_table, \
                bt_stride, bt_rows, NH, NKV, page_size, num_pages, scale, window, n_splits, part_acc, part_ml, counters, max_kv, \
                cluster_merge, stream
    switch (D) {
        case 64: return launch_decode<64>(AD_ARGS);
        case 128: return launch_decode<128>(AD_ARGS);
        default: return ACV_ERR_SIZE;
    }
#undef AD_ARGS
}

// How many CTAs of the split-KV kernel the device holds at once for these sizes (clusters that fit, times their size,
// when the splits merge inside clusters): what the choice of the number of splits is made from.  With ``alone``: how many
// it holds one to an SM, which is the largest grid that runs with eight warps to a CTA (0: that form does not fit these
// sizes).  Negative: an error.
ACV_API int acv_attention_decode_resident(int NH, int NKV, int D, int page_size, int window, int n_splits, int max_kv,
                                          int cluster_merge, int alone) {
    if (NKV <= 0 || NH % NKV || NH / NKV > 16 || n_splits < 1 || n_splits > 65535 || page_size <= 0) return ACV_ERR_SIZE;
    if (D != 64 && D != 128) return ACV_ERR_SIZE;
    if (n_splits < 2 || n_splits > 8) cluster_merge = 0;
    int pg_cap = 0;
    const int cluster = cluster_merge ? n_splits : 1;
    if (alone) {
        int alone_bytes = 0, dev = 0, per_block = 0;
        const bool any = D == 64 ? decode_grid_has_sms<64>(cluster, 1, &alone_bytes) : decode_grid_has_sms<128>(cluster, 1, &alone_bytes);
        if (!any) return 0;
        const int smem = decode_smem_bytes(D, NH / NKV, page_size, window, n_splits, max_kv, cluster_merge, AD_WARPS_ALONE, &pg_cap);
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&per_block, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) {
            cudaGetLastError();
            return ACV_ERR_SIZE;
        }
        if (smem > per_block) return 0;
        const int use = smem < alone_bytes ? alone_bytes : smem;
        return D == 64 ? decode_resident<64, AD_WARPS_ALONE>(use, cluster) : decode_resident<128, AD_WARPS_ALONE>(use, cluster);
    }
    const int smem = decode_smem_bytes(D, NH / NKV, page_size, window, n_splits, max_kv, cluster_merge, AD_WARPS, &pg_cap);
    return D == 64 ? decode_resident<64, AD_WARPS>(smem, cluster) : decode_resident<128, AD_WARPS>(smem, cluster);
}

// ----------------------------------------------------------------------------- entry point without allocation
// See no_alloc.h.  The split-KV kernel needs scratch for the partial results of the splits; here it
// lives in a file-scope device array of fixed size instead of memory the caller allocates.
#include "no_alloc.h"

#define AD_STATIC_FLOATS (1 << 20)   /* 4 MiB on every GPU that loads this library, until the process exits */
static __device__ __align__(256) float ad_static_scratch[AD_STATIC_FLOATS];

// In host code `ad_static_scratch` is only a handle for the runtime; the device address has to be
// asked for, once per device, with that device current.
static float* ad_static_address(int* error) {
    static float* address[64] = {nullptr};
    static std::mutex lock;                     // host threads may make their first calls side by side
    std::lock_guard<std::mutex> guard(lock);
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= 64) {
        *error = e != cudaSuccess ? (int)e : ACV_ERR_SIZE;
        return nullptr;
    }
    if (!address[device]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, ad_static_scratch);
        if (e != cudaSuccess) {
            *error = (int)e;
            return nullptr;
        }
        address[device] = (float*)p;
    }
    *error = 0;
    return address[device];
}

ACV_API long long acv_attention_decode_static_capacity(void) { return AD_STATIC_FLOATS; }

ACV_API int acv_attention_decode_static(const void* q, int q_stride, void* out, int out_stride, const void* k_pages,
                                        const void* v_pages, const int* dec_tokens, const int* dec_seqs, int n_dec,
                                        const int* kv_len, const int* block_table, int bt_stride, int NH, int NKV,
                                        int D, int page_size, int num_pages, float scale, int window, int n_splits,
                                        int max_kv, cudaStream_t stream) {
    if (n_dec <= 0) return 0;
    if (NKV <= 0 || NH % NKV || n_splits < 1) return ACV_ERR_SIZE;
    const long long n_rep = NH / NKV;
    const long long parts = n_splits > 1 ? (long long)n_dec * NKV * n_splits : 0;
    const long long acc_floats = parts * n_rep * D;
    const long long ml_floats = parts * n_rep * 2;
    const long long counters = (long long)n_dec * NKV;
    // layout inside the array: [partial accumulators | partial (max, sum) | one counter per (request, kv-head)]
    if (acc_floats + ml_floats + counters > AD_STATIC_FLOATS) return ACV_ERR_SCRATCH;
    int error = 0;
    float* base = ad_static_address(&error);
    if (!base) return error;
    float* part_acc = base;
    float* part_ml = base + acc_floats;
    int* cnt = reinterpret_cast<int*>(base + acc_floats + ml_floats);
    // the array keeps what the last call left, and a call with another shape puts its counters
    // elsewhere: the counters of this call are cleared on the stream before the kernel runs
    cudaError_t e = cudaMemsetAsync(cnt, 0, (size_t)counters * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
    return acv_attention_decode(q, q_stride, out, out_stride, k_pages, v_pages, dec_tokens, dec_seqs, n_dec, kv_len,
                                block_table, bt_stride, nullptr, NH, NKV, D, page_size, num_pages, scale, window, n_splits,
                                part_acc, part_ml, cnt, acc_floats, ml_floats, counters, max_kv, 0, stream);
}

ACV_TL_EXPORT(attention_decode)
