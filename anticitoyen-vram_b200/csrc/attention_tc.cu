// Paged causal flash attention for portions of prompts on the fifth-generation tensor cores.
//
// One CTA per (tile of 128 query tokens of one request, pair of query heads that share a key/value
// head).  The two heads see the same keys, the same values and the same mask, so a tile of 128 keys is
// loaded once for both.  Each head works through a tile of keys in two halves of 64, a and b:
//   S_x = Q_h K_x^T  tcgen05.mma, Q and K in shared memory (K-major, 128-byte swizzle), S_x in 64 columns of
//                    tensor memory of its own
//   softmax          four warps per head, one query row per thread: the row of S_x from tensor memory
//                    (tcgen05.ld), mask by absolute position, running maximum and sum in float; P_x goes
//                    back into the first columns of S_x as packed bfloat16 (tcgen05.st), the A operand of the
//                    next product; the row of O_h in tensor memory is rescaled only when its maximum has grown
//                    by more than 2^8 since the last rescale (the sum and O carry the same stale maximum,
//                    so the quotient at the end is unchanged)
//   O_h += P_x V_x   tcgen05.mma with A from tensor memory, V in shared memory as it lies in the pages
//                    ([keys][D], the MN-major operand)
// Each head has an issuing thread of its own.  When the softmax hands over P_x it issues P_x.V_x and then S_x of the
// next tile of keys; products of one thread run in the order of issue, so the next S_x overwrites P_x only after
// P_x.V_x has read it.  While the softmax warps work on one half, the scores of the other half are already there or on
// their way: they do not wait for the tensor core between halves, and the tensor core has one head's products to
// run while the other head's warps take their exponentials.  A row's O is rescaled only while no product on values
// of its head is in flight (the issuing thread commits each to a barrier that the softmax warps wait on then).
// Keys and values come straight from the cache pages by TMA, one box per page and 64 columns, two
// tiles in flight, keys and values in rings of their own; Q comes by TMA from the step's projection buffer.  Warp 0
// issues the loads, warps 1 and 10 the MMAs of head 0 and head 1, warps 2..5 are head 0's softmax and epilogue,
// warps 6..9 head 1's.  A group with an odd
// number of query heads leaves the second half of its last CTA idle.  The mask follows absolute positions
// (key j is seen by the query at position p iff j <= p, and j > p - window when a window is set), so a
// portion may start anywhere in its prompt (acvram/engine/layers.py:1020-1041); the reference runs this
// case through SDPA on a gathered dense copy (acvram/engine/attention.py:519-584).
// Every wait is bounded; a wait that runs out is recorded in `status` and the kernel returns.
#include "tc_ptx.cuh"
#include "tensor_map.h"

#define AT_THREADS 352
#define AT_BM 128
#define AT_BN 128
#define AT_LOG2E 1.4426950408889634f
#define AT_ATOM (128 * 128)          // bytes of one swizzle atom column: 128 rows of 128 bytes
#define AT_HALF 64                   // keys of a half tile
#define AT_LAZY 8.0f                 // a row's maximum may lag by this much (log2 units) before O is rescaled

struct AttnTcParams {
    bf16* out;
    int out_stride;
    const int* tile_seq;
    const int* tile_q0;
    const int* cu_q;
    const int* kv_len;
    const int* block_table;
    int bt_stride;
    const int* bt_rows;         // the row of block_table of each request of the batch (null: its index)
    int NH, NKV, page_size, page_shift, num_pages, window;
    float scale;
    int* status;
};

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, AttnTcParams p) {
    constexpr int DA = D / 64;                         // 64-element column atoms of a head
    constexpr int Q_BYTES = DA * AT_ATOM, KV_BYTES = DA * AT_ATOM;
    constexpr int TMEM_COLS = 512;                     // S_h,x: columns [128h + 64x, + 64), O_h: [256 + 128h, 256 + 128h + D)
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = smem_raw + ((1024u - (gt_smem(smem_raw) & 1023u)) & 1023u);
    const uint32_t q_s = gt_smem(base), kv_s = q_s + 2 * Q_BYTES;   // q_s: [2 heads]; kv_s: [2 stages][K, V]
    uint64_t* bars = (uint64_t*)(base + 2 * Q_BYTES + 4 * KV_BYTES);       // 21 barriers
    const uint32_t bar0 = gt_smem(bars);
    // keys and values have rings of their own: a tile's keys are free once both heads' scores are issued, long before
    // its values are (after both heads' second P.V)
    const uint32_t q_full = bar0, k_full = bar0 + 8, k_free = bar0 + 24, v_full = bar0 + 40, v_free = bar0 + 56,
                   s_full = bar0 + 72 /*[head][half]*/, p_full = bar0 + 104 /*[head][half]*/, o_full = bar0 + 136 /*[head]*/,
                   pv_done = bar0 + 152 /*[head]*/;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ACV_TL(TL_ATTN_TC, 64);
    // the CTA's heads, from its number alone (the barriers' counts depend on it)
    const int n_rep = p.NH / p.NKV, pairs = (n_rep + 1) >> 1;
    const int tile = blockIdx.x / (p.NKV * pairs), hp = blockIdx.x - tile * (p.NKV * pairs);
    const int kvh = hp / pairs, pair = hp - kvh * pairs;
    const int h0 = kvh * n_rep + 2 * pair;                  // the CTA's first head; the second is h0 + 1
    const int n_heads = 2 * pair + 1 < n_rep ? 2 : 1;
    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(k_full + 8 * s, 1); mbar_init(k_free + 8 * s, n_heads);      // each head's issuing thread frees
            mbar_init(v_full + 8 * s, 1); mbar_init(v_free + 8 * s, n_heads);
        }
        for (int i = 0; i < 4; ++i) { mbar_init(s_full + 8 * i, 1); mbar_init(p_full + 8 * i, 4); }
        for (int h = 0; h < 2; ++h) { mbar_init(o_full + 8 * h, 1); mbar_init(pv_done + 8 * h, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(&tmem_base_s)), "r"(TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    // The key/value ring starts at zero: a page that is skipped (every key of it masked) leaves its rows
    // as they were, and a masked key's value is multiplied by a zero probability, so it must be finite.
    for (int i = threadIdx.x; i < 4 * KV_BYTES / 16; i += AT_THREADS)
        reinterpret_cast<uint4*>(base + 2 * Q_BYTES)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_base_s;
    // only now may the next kernel's CTAs come: one that took tensor memory before this CTA had its own
    // would wait for this grid to end while this CTA waits for its columns
    pdl_launch_dependents();

    // ---- the tile's geometry (the same in every role), from the step's index arrays, which were written before the
    // step's first kernel began: read while the projection before this kernel still runs
    // blocks are numbered tile-major: the tile list begins with the longest tiles, and the hardware hands
    // out blocks in the order of their numbers, so every head pair of a long tile starts before a short one
    const int seq = p.tile_seq[tile], q0 = p.tile_q0[tile];
    const int tok0 = p.cu_q[seq] + q0;
    const int q_len = p.cu_q[seq + 1] - p.cu_q[seq];
    const int rows = min(AT_BM, q_len - q0);
    const int pos0 = p.kv_len[seq] - q_len + q0;            // absolute position of the tile's first query
    const int hi = pos0 + rows - 1;                         // last key any row sees
    const int lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int j_first = lo & ~(AT_BN - 1);
    const int n_tiles = (hi - j_first) / AT_BN + 1;
    const int* bt = p.block_table + (size_t)(p.bt_rows ? p.bt_rows[seq] : seq) * p.bt_stride;
    pdl_wait();             // queries, and the keys and values of this step's tokens, are the projection's output

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // lane i brings page i of a key tile, so the block-table reads of a tile's pages run side by side
        if (lane == 0) {
            mbar_expect_tx(q_full, n_heads * Q_BYTES);
            for (int h = 0; h < n_heads; ++h)
#pragma unroll
                for (int a = 0; a < DA; ++a)
                    tma_load_2d(q_s + h * Q_BYTES + a * AT_ATOM, &map_q, q_full, (h0 + h) * D + a * 64, tok0);
        }
        const int ps = p.page_size, pages_per_tile = AT_BN >> p.page_shift;
        for (int t = 0; t < n_tiles; ++t) {
            const int s = t & 1;
            // pages of this tile that hold keys some row reads; the others are skipped (their rows are masked)
            const int j = j_first + t * AT_BN + lane * ps;
            int pg = -1;
            if (lane < pages_per_tile && j <= hi && j + ps - 1 >= lo) pg = bt[j >> p.page_shift];
            const bool take = pg >= 0 && pg < p.num_pages;
            const uint32_t taken = __ballot_sync(0xffffffffu, take);
            const uint32_t k_dst = kv_s + s * 2 * KV_BYTES + lane * ps * 128, v_dst = k_dst + KV_BYTES;
            const int row = (pg * p.NKV + kvh) * ps;
            bool stop = false;
            for (int kv = 0; kv < 2 && !stop; ++kv) {           // the keys, then the values
                const uint32_t full = (kv ? v_full : k_full) + 8 * s, free_bar = (kv ? v_free : k_free) + 8 * s;
                int go = 1;
                if (lane == 0) {
                    if (abort_s) go = 0;
                    else if (t >= 2 && !mbar_wait(free_bar, ((t >> 1) - 1) & 1, &abort_s)) {
                        abort_s = 1; atomicExch(p.status, 11); go = 0;
                    }
                    if (go) mbar_expect_tx(full, __popc(taken) * (uint32_t)DA * ps * 128u);
                }
                if (!__shfl_sync(0xffffffffu, go, 0)) { stop = true; break; }
                if (take) {
#pragma unroll
                    for (int a = 0; a < DA; ++a)
                        tma_load_2d((kv ? v_dst : k_dst) + a * AT_ATOM, kv ? &map_v : &map_k, full, a * 64, row);
                }
            }
            if (stop) break;
        }
    } else if (warp == 1 || warp == 10) {
        // ------------------------------------------------------------------ MMA issuers: warp 1 for head 0, warp 10 for head 1
        const int h = warp == 1 ? 0 : 1;
        if (lane == 0 && h < n_heads) {
            const uint32_t idesc_s = umma_idesc(AT_HALF, 128, 0), idesc_o = umma_idesc(D, 128, 1);
            const uint32_t q_lo = umma_desc_lo(q_s + h * Q_BYTES);
            // S_x = Q_h K_x^T over the head dimension, for half x of the tile of keys in stage s (the half's 64 key rows
            // lie 64 x 128 bytes into each column atom)
            auto issue_s = [&](int x, int s) {
                const uint32_t k_lo = umma_desc_lo(kv_s + s * 2 * KV_BYTES + x * (AT_HALF * 128));
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk) {
                    const uint32_t off = ((kk >> 2) * AT_ATOM + (kk & 3) * 32) >> 4;
                    tc_mma_bf16_h(tmem + h * 128 + x * AT_HALF, q_lo + off, k_lo + off, idesc_s, kk > 0 ? 1u : 0u);
                }
                tc_commit(s_full + 8 * (2 * h + x));
            };
            bool ok = mbar_wait(q_full, 0, &abort_s);
            if (!ok) { abort_s = 1; atomicExch(p.status, 12); }
            if (ok && !mbar_wait(k_full, 0, &abort_s)) { ok = false; abort_s = 1; atomicExch(p.status, 13); }
            if (ok) {
                tc_fence_after();
                issue_s(0, 0);
                issue_s(1, 0);
                tc_commit(k_free);                  // this head has read the first tile's keys
            }
            for (int t = 0; t < n_tiles && ok && !abort_s; ++t) {
                const int s = t & 1;
                const uint32_t v_lo = umma_desc_lo(kv_s + s * 2 * KV_BYTES + KV_BYTES, AT_ATOM);
                for (int x = 0; x < 2 && ok; ++x) {
                    // O_h += P_x V_x over the half's keys, once the softmax has written P_x
                    if (!mbar_wait(p_full + 8 * (2 * h + x), t & 1, &abort_s)) { ok = false; abort_s = 1; atomicExch(p.status, 14); break; }
                    if (x == 0 && !mbar_wait(v_full + 8 * s, (t >> 1) & 1, &abort_s)) { ok = false; abort_s = 1; atomicExch(p.status, 13); break; }
                    tc_fence_after();
#pragma unroll
                    for (int k4 = 0; k4 < AT_HALF / 16; ++k4)
                        tc_mma_bf16_ts_h(tmem + 256 + h * 128, tmem + h * 128 + x * AT_HALF + k4 * 8,
                                         v_lo + (x * (AT_HALF / 16) + k4) * (2048 >> 4), idesc_o, (t > 0 || x > 0 || k4 > 0) ? 1u : 0u);
                    tc_commit(pv_done + 8 * h);                     // O_h is at rest again when this arrives
                    if (x == 1) tc_commit(v_free + 8 * s);         // this head has read the stage's values
                    if (t + 1 < n_tiles) {
                        if (x == 0) {
                            if (!mbar_wait(k_full + 8 * (s ^ 1), ((t + 1) >> 1) & 1, &abort_s)) { ok = false; abort_s = 1; atomicExch(p.status, 13); break; }
                            tc_fence_after();
                        }
                        issue_s(x, s ^ 1);
                        if (x == 1) tc_commit(k_free + 8 * (s ^ 1));
                    }
                }
            }
            tc_commit(o_full + 8 * h);
        }
    } else if (((warp - 2) >> 2) < n_heads) {
        // ------------------------------------------------------------------ softmax and epilogue of one head
        const int hs = (warp - 2) >> 2;                         // head slot 0 or 1
        const int wq = warp & 3;                                // the tensor-memory lanes this warp may touch
        const int r = wq * 32 + lane;                           // this thread's query row = tensor-memory lane
        const int pos = pos0 + r;
        const uint32_t lane_base = (uint32_t)(wq * 32) << 16;
        const uint32_t tmem_s = tmem + hs * 128 + lane_base, tmem_o = tmem + 256 + hs * 128 + lane_base;
        const float scale_log2 = p.scale * AT_LOG2E;
        float m_run = -INFINITY, l_run = 0.f;
        bool failed = false;
#ifdef ACV_TIMELINE
        unsigned long long tl_acc[5] = {0, 0, 0, 0, 0}, tl_t = acv_tl_now();
#define TL_PHASE(i) do { const unsigned long long n_ = acv_tl_now(); tl_acc[i] += n_ - tl_t; tl_t = n_; } while (0)
#else
#define TL_PHASE(i)
#endif
        for (int tx = 0; tx < 2 * n_tiles && !abort_s; ++tx) {
            const int t = tx >> 1, x = tx & 1;                  // tile of keys and its half
            if (!mbar_wait(s_full + 8 * (2 * hs + x), t & 1, &abort_s)) { abort_s = 1; atomicExch(p.status, 15); failed = true; break; }
            tc_fence_after();
            TL_PHASE(0);
            const uint32_t tmem_sx = tmem_s + x * AT_HALF;
            const int j0 = j_first + t * AT_BN + x * AT_HALF;
            const bool need_mask = j0 + AT_HALF - 1 > pos0 || (p.window > 0 && j0 <= pos0 + AT_BM - 1 - p.window);
            uint32_t ra[32], rb[32];
            auto masked = [&](uint32_t (&raw)[32], int c0) {
#pragma unroll
                for (int c = 0; c < 32; ++c) {
                    const int j = j0 + c0 + c;
                    const bool seen = j <= pos && (p.window <= 0 || j > pos - p.window);
                    raw[c] = seen ? raw[c] : 0xff800000u;       // -inf
                }
            };
            // first pass: the row's maximum over the half's 64 scores
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            tc_ld32_nowait(tmem_sx, ra);
            tc_ld32_nowait(tmem_sx + 32, rb);
            tc_wait_ld();
            if (need_mask) { masked(ra, 0); masked(rb, 32); }
#pragma unroll
            for (int c = 0; c < 32; ++c) mx4[c & 3] = fmaxf(mx4[c & 3], fmaxf(__uint_as_float(ra[c]), __uint_as_float(rb[c])));
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
            TL_PHASE(1);
            // the maximum in use moves only when the true one has run ahead of it by more than AT_LAZY
            const float m_true = fmaxf(m_run, mx * scale_log2);
            float alpha = 1.f;
            if (m_true > m_run + AT_LAZY) {         // also the first finite maximum of a row (-inf + 8 = -inf)
                alpha = m_run == -INFINITY ? 0.f : tc_exp2(m_run - m_true);
                m_run = m_true;
            }
            const float m_use = m_run == -INFINITY ? 0.f : m_run;
            // rows whose maximum moved rescale what O holds so far (tensor-memory access is warp-wide).  O has to be at
            // rest: the product on values issued last for this head, number tx - 1, must be complete (the one before it
            // is, since this half's scores were issued after it, and the next waits for this half's P)
            if (tx > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
                if (!mbar_wait(pv_done + 8 * hs, (tx - 1) & 1, &abort_s)) { abort_s = 1; atomicExch(p.status, 17); failed = true; break; }
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < D; c0 += 32) {
                    uint32_t o[32];
                    tc_ld32(tmem_o + c0, o);
#pragma unroll
                    for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                    tc_st32(tmem_o + c0, o);
                }
            }
            l_run *= alpha;
            TL_PHASE(2);
            // second pass, on the scores still in registers: P = 2^(s * scale - m) as packed bfloat16 into the first 32
            // columns of S_x
            auto exp_of = [&](uint32_t (&raw)[32], int c0) {
                float part[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t pk[16];
#pragma unroll
                for (int c = 0; c < 32; c += 2) {
                    const float e0 = tc_exp2(fmaf(__uint_as_float(raw[c]), scale_log2, -m_use));
                    const float e1 = tc_exp2(fmaf(__uint_as_float(raw[c + 1]), scale_log2, -m_use));
                    part[c & 3] += e0;
                    part[(c + 1) & 3] += e1;
                    pk[c >> 1] = pack_bf16x2(e0, e1);
                }
                l_run += (part[0] + part[1]) + (part[2] + part[3]);
                tc_st16_nowait(tmem_sx + (c0 >> 1), pk);
            };
            exp_of(ra, 0);
            exp_of(rb, 32);
            TL_PHASE(3);
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(p_full + 8 * (2 * hs + x));
            TL_PHASE(4);
        }
#ifdef ACV_TIMELINE
        if (threadIdx.x == 64) {
            for (int i = 0; i < 5; ++i) acv_tl_marks[i] = tl_acc[i];
            acv_tl_marks[7] = (unsigned long long)(2 * n_tiles);
        }
#endif
        if (!failed && !abort_s && mbar_wait(o_full + 8 * hs, 0, &abort_s)) {
            tc_fence_after();
            const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
            bf16* dst = p.out + (size_t)(tok0 + r) * p.out_stride + (size_t)(h0 + hs) * D;
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t o[32];
                tc_ld32(tmem_o + c0, o);
                if (r < rows) {
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 pk;
                        pk.x = pack_bf16x2(__uint_as_float(o[c]) * inv, __uint_as_float(o[c + 1]) * inv);
                        pk.y = pack_bf16x2(__uint_as_float(o[c + 2]) * inv, __uint_as_float(o[c + 3]) * inv);
                        pk.z = pack_bf16x2(__uint_as_float(o[c + 4]) * inv, __uint_as_float(o[c + 5]) * inv);
                        pk.w = pack_bf16x2(__uint_as_float(o[c + 6]) * inv, __uint_as_float(o[c + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + c) = pk;
                    }
                }
            }
        } else if (!failed && !abort_s) {
            abort_s = 1;
            atomicExch(p.status, 16);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base_s), "r"(TMEM_COLS));
    }
}

template <int D>
static int launch_attn_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const AttnTcParams& p,
                          int n_tiles, cudaStream_t stream) {
    constexpr int SMEM = 2 * (D / 64) * AT_ATOM /*Q of two heads*/ + 4 * (D / 64) * AT_ATOM /*K,V x2*/ + 1024 + 256;
    static AcvSmemConfig smem_config;          // per kernel instance and device
    if (int rc = acv_ensure_smem(smem_config, attn_tc_kernel<D>, SMEM)) return rc;
    const int n_rep = p.NH / p.NKV;
    acv_launch(PDL_MISC, attn_tc_kernel<D>, dim3((unsigned)(n_tiles * (p.NKV * ((n_rep + 1) / 2)))), AT_THREADS, SMEM, stream, mq, mk, mv, p);
    return acv_launch_status();
}

// q: the step's stacked projection [T, q_width] (queries are its first NH*D columns, row stride q_stride);
// pages [num_pages, NKV, page_size, D]; tile lists as for the tiled kernel, with tiles of 128 query tokens.
// Takes head sizes 64 and 128 and page sizes that are powers of two from 8 to 128.
ACV_API int acv_attention_tc(const void* q, int q_stride, int T, void* out, int out_stride, const void* k_pages,
                             const void* v_pages, const int* tile_seq, const int* tile_q0, int n_tiles, const int* cu_q,
                             const int* kv_len, const int* block_table, int bt_stride, const int* bt_rows, int NH, int NKV,
                             int D, int page_size, int num_pages, float scale, int window, int* status, cudaStream_t stream) {
    if (n_tiles <= 0) return 0;
    if (NKV <= 0 || NH % NKV || NH > 65535 || (D != 64 && D != 128)) return ACV_ERR_SIZE;
    if ((long long)n_tiles * NH > 0x7fffffffLL) return ACV_ERR_SIZE;
    int page_shift = -1;
    for (int b = 3; b <= 7; ++b)
        if ((1 << b) == page_size) page_shift = b;
    if (page_shift < 0) return ACV_ERR_SIZE;
    if (((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
        ((uintptr_t)out & 15) || (out_stride % 8))
        return ACV_ERR_ALIGN;
    CUtensorMap mq, mk, mv;
    int rc = make_map(&mq, q, T, NH * D, q_stride, AT_BM);
    if (rc) return rc;
    const long long pool_rows = (long long)num_pages * NKV * page_size;
    if (pool_rows > 0x7fffffffLL) return ACV_ERR_SIZE;
    rc = make_map(&mk, k_pages, (int)pool_rows, D, D, page_size);
    if (rc) return rc;
    rc = make_map(&mv, v_pages, (int)pool_rows, D, D, page_size);
    if (rc) return rc;
    AttnTcParams p;
    p.out = (bf16*)out; p.out_stride = out_stride; p.tile_seq = tile_seq; p.tile_q0 = tile_q0; p.cu_q = cu_q;
    p.kv_len = kv_len; p.block_table = block_table; p.bt_stride = bt_stride; p.bt_rows = bt_rows; p.NH = NH; p.NKV = NKV;
    p.page_size = page_size; p.page_shift = page_shift; p.num_pages = num_pages; p.window = window; p.scale = scale;
    p.status = status;
    if (D == 64) return launch_attn_tc<64>(mq, mk, mv, p, n_tiles, stream);
    return launch_attn_tc<128>(mq, mk, mv, p, n_tiles, stream);
}

ACV_TL_EXPORT(attention_tc)
