// C[M,N] = X[M,K] . W[N,K]^T in bfloat16 on the fifth-generation tensor cores:
// tcgen05.mma with both operands in shared memory (staged by TMA, 128-byte
// swizzle) and the accumulator in tensor memory, read back with tcgen05.ld.
//
// One kernel serves prefill and decode.  An MMA tile is 128 rows of the "A
// operand" by BN rows of the "B operand", both K-major, which is how x [M,K] and
// a weight [N,K] both lie in memory.  With many tokens the tokens are the A
// operand (128 tokens x BN features per tile); with few tokens (decode) the roles
// are swapped: 128 output features x BN tokens per tile, so that every weight is
// streamed from memory once whatever the batch and the tensor core's M = 128 is
// filled by the weight rows.  The K range may be split over several CTAs (decode
// has too few tiles to fill 148 SMs otherwise); partial tiles go to a float
// workspace and the CTA that arrives last at a tile adds them in split order, so
// the sum does not depend on timing.  The reference hands these products to cuBLAS
// (acvram/kernels/__init__.py:1896-1899).
//
// Warp roles in a CTA of 192 threads: warp 0 issues the TMA loads, warp 1
// allocates tensor memory and issues the MMAs (one thread each), warps 2..5 are
// the epilogue (each owns the 32 accumulator lanes its rank modulo 4 may read).
// A CTA walks its work items with a fixed stride, two accumulator buffers in
// tensor memory let the epilogue of one item overlap the main loop of the next.
// Every wait on an mbarrier is bounded: when a wait runs out, the kernel records
// where in `status`, all roles leave their loops, tensor memory is freed and the
// kernel returns.
#include <mutex>

#include "common.cuh"

#define GT_THREADS 192

#include "gemm_epilogue.cuh"
#include "tensor_map.h"

// The q,k,v epilogue with tokens on the tensor-memory lanes (many tokens, features on columns): a thread holds one
// token's row of the tile, whole heads of it, so norm and rotation stay inside the thread.  Head by head: the
// head's D columns are read from tensor memory and rounded to bfloat16 (what the projection's output would hold),
// their squares summed; then, 16 angles at a time, both halves of the head are scaled, rotated and written: queries to
// C, keys and values to the token's page.  The same arithmetic as gt_flush_qkv and the rotation kernel.
template <int BN, int D>                         // D: head size, 64 or 128; BN is a multiple of it
__device__ __forceinline__ void gt_store_qkv_rows(const GemmParams& p, uint32_t taddr, int token, int tb) {
    const bool live = token < p.M;
    int pos = 0, pg = -1;
    if (live) {
        pos = p.positions[token];
        {
            const int sq = p.seq_of_token[token];
            pg = p.block_table[(size_t)(p.bt_rows ? p.bt_rows[sq] : sq) * p.bt_stride + pos / p.page_size];
        }
        if (pg >= p.num_pages) pg = -1;
    }
    const bool in_table = pos >= 0 && pos < p.table_rows;
    const float* cs = p.cos_sin ? p.cos_sin + (size_t)(in_table ? pos : 0) * D : nullptr;
#pragma unroll 1
    for (int h0 = 0; h0 < BN; h0 += D) {
        const int f0 = tb * BN + h0;                // first feature of the head in the stacked output
        if (f0 >= p.N) break;
        const int head = f0 / D;
        const bool is_q = head < p.q_heads, is_k = !is_q && head < p.q_heads + p.kv_heads, is_v = !is_q && !is_k;
        const float* w = is_q ? p.q_w : (is_k ? p.k_w : nullptr);
        // the head's values, rounded as the projection rounds, kept as pairs
        uint32_t packed[D / 2];
        float ss = 0.f;
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 16) {
            {                                       // tensor-memory loads are executed by whole warps
                uint32_t r[16];
                tc_ld16(taddr + h0 + c0, r);
#pragma unroll
                for (int c = 0; c < 16; c += 2) {
                    const uint32_t pk = pack2(r[c], r[c + 1]);
                    packed[(c0 + c) >> 1] = pk;
                    const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&pk);
                    const float x0 = __low2float(b2), x1 = __high2float(b2);
                    ss += x0 * x0 + x1 * x1;
                }
            }
        }
        const float inv = w ? rsqrtf(ss / (float)D + p.qk_eps) : 1.f;
        bf16* dst = nullptr;
        if (live) {
            if (is_q) {
                dst = (bf16*)p.C + (size_t)token * p.ldc + f0;
            } else if (pg >= 0) {
                const int kvh = is_k ? head - p.q_heads : head - p.q_heads - p.kv_heads;
                dst = (is_k ? p.k_pages : p.v_pages) + (((size_t)pg * p.kv_heads + kvh) * p.page_size + (pos % p.page_size)) * D;
            }
        }
        const bool rotate = cs && !is_v && in_table;
        constexpr int half = D >> 1;
#pragma unroll
        for (int i0 = 0; i0 < half; i0 += 16) {
            {
                float lo[16], hi[16];               // elements i0 .. i0+15 and their partners half further
#pragma unroll
                for (int c = 0; c < 16; c += 2) {
                    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&packed[(i0 + c) >> 1]);
                    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&packed[(half + i0 + c) >> 1]);
                    lo[c] = __low2float(a); lo[c + 1] = __high2float(a);
                    hi[c] = __low2float(b); hi[c + 1] = __high2float(b);
                }
                if (w) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        lo[c] = lo[c] * inv * __ldg(w + i0 + c);
                        hi[c] = hi[c] * inv * __ldg(w + half + i0 + c);
                    }
                }
                if (rotate) {
#pragma unroll
                    for (int c4 = 0; c4 < 16; c4 += 4) {
                        const float4 c = *reinterpret_cast<const float4*>(cs + i0 + c4);
                        const float4 sn = *reinterpret_cast<const float4*>(cs + half + i0 + c4);
                        const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                        for (int u = 0; u < 4; ++u) {
                            const float a = lo[c4 + u], b = hi[c4 + u];
                            lo[c4 + u] = a * cc[u] - b * sv[u];
                            hi[c4 + u] = b * cc[u] + a * sv[u];
                        }
                    }
                }
                if (dst) {
                    uint4 o;
#pragma unroll
                    for (int g = 0; g < 2; ++g) {
                        o.x = pack2(__float_as_uint(lo[8 * g]), __float_as_uint(lo[8 * g + 1]));
                        o.y = pack2(__float_as_uint(lo[8 * g + 2]), __float_as_uint(lo[8 * g + 3]));
                        o.z = pack2(__float_as_uint(lo[8 * g + 4]), __float_as_uint(lo[8 * g + 5]));
                        o.w = pack2(__float_as_uint(lo[8 * g + 6]), __float_as_uint(lo[8 * g + 7]));
                        *reinterpret_cast<uint4*>(dst + i0 + 8 * g) = o;
                        o.x = pack2(__float_as_uint(hi[8 * g]), __float_as_uint(hi[8 * g + 1]));
                        o.y = pack2(__float_as_uint(hi[8 * g + 2]), __float_as_uint(hi[8 * g + 3]));
                        o.z = pack2(__float_as_uint(hi[8 * g + 4]), __float_as_uint(hi[8 * g + 5]));
                        o.w = pack2(__float_as_uint(hi[8 * g + 6]), __float_as_uint(hi[8 * g + 7]));
                        *reinterpret_cast<uint4*>(dst + half + i0 + 8 * g) = o;
                    }
                }
            }
        }
    }
}

template <int BN>
struct GemmShape {
    static constexpr int STAGE_BYTES = (GT_BM + BN) * GT_BK * 2;
    static constexpr int MAX_STAGES = (200 * 1024 / STAGE_BYTES) > 8 ? 8 : (200 * 1024 / STAGE_BYTES);
    // two accumulator buffers side by side; tensor memory is given out in powers of two of columns
    static constexpr int TMEM_COLS = 2 * BN <= 32 ? 32 : 2 * BN <= 64 ? 64 : 2 * BN <= 128 ? 128 : 2 * BN <= 256 ? 256 : 512;
    static constexpr int PART_BYTES = BN * GT_BM * 4;                 // one CTA's partial tile in float
    static constexpr int smem_bytes(int stages, int cluster_parts, int aux_bytes = 0) {
        return stages * STAGE_BYTES + 1024 /*align*/ + 256 /*barriers*/ + cluster_parts * PART_BYTES + aux_bytes;
    }
};

// Which tile a work item is.  Tiles are walked in groups of `group` rows of tiles (all columns of a group before the
// next group), rows fastest: the CTAs that run at one time then share few rows of tiles and a few columns of
// them, so that with many tokens neither the activations nor the weights are read from memory over and over.
__device__ __forceinline__ void gt_tile_of(int tile, int tiles_a, int tiles_b, int group, int& ta, int& tb) {
    if (group >= tiles_a) {         // one group (weights on the rows): a single division, the thread that loads is waited for
        tb = tile / tiles_a;
        ta = tile - tb * tiles_a;
        return;
    }
    const int per_group = group * tiles_b;
    const int g = tile / per_group, r = tile - g * per_group;
    const int rows = min(group, tiles_a - g * group);
    tb = r / rows;
    ta = g * group + (r - tb * rows);
}

// Registers are handed out to a CTA for its warps rounded up to four: 192 threads count as 8 warps, and three
// such CTAs share an SM (what the narrow decode products with short pipelines want) only up to 80 registers
// a thread (measured: at 106 registers two came to an SM and the gate/up product of a decode step ran in
// two waves).  The narrow tile is held to that; the wider ones never come three to an SM.
template <int BN>
__global__ void __launch_bounds__(GT_THREADS, 1) __maxnreg__(BN <= 16 ? 80 : 232)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    using S = GemmShape<BN>;
    extern __shared__ unsigned char smem_raw[];
    // operand tiles start on a 1024-byte boundary of the shared window (the swizzle pattern is anchored there)
    unsigned char* tiles = smem_raw + ((1024u - (gt_smem(smem_raw) & 1023u)) & 1023u);
    const int STAGES = p.stages;
    uint64_t* bars = (uint64_t*)(tiles + STAGES * S::STAGE_BYTES);
    // bars: full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]
    const uint32_t full0 = gt_smem(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;
    const uint32_t part_bar = tempty0 + 16;         // rank 0 of a split's cluster: counts the bytes of the peers' partial tiles
    const uint32_t part0 = gt_smem(tiles) + STAGES * S::STAGE_BYTES + 256;     // [splits-1][BN][128] floats (cluster mode)
    const bool cluster_split = p.cluster && p.splits > 1;
    // the q,k,v epilogue's tables lie behind the partial tiles
    unsigned char* aux = tiles + STAGES * S::STAGE_BYTES + 256 + (cluster_split ? (p.splits - 1) * S::PART_BYTES : 0);
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;
    __shared__ volatile int never_s;            // stays 0: for the one wait that the CTA's own failure must not cut short
    __shared__ int last_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    ACV_TL(TL_GEMM, 64);
    if (threadIdx.x == 0) {
        abort_s = 0;
        never_s = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
        mbar_init(part_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // rank 0 of a split's cluster announces the peers' partial tiles at once (their bytes may come before or after)
        if (cluster_split && cluster_ctarank() == 0) mbar_expect_tx(part_bar, (uint32_t)(p.splits - 1) * S::PART_BYTES);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(&tmem_base_s)), "r"(S::TMEM_COLS));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    // only now may the next kernel's CTAs come: one that took tensor memory before this CTA had its own
    // could wait for this grid to end while this CTA waits for its columns
    pdl_launch_dependents();
    // split K inside a cluster: ranks 1.. write their partial tiles into rank 0's shared memory at the end.  They may
    // do so only when they know that rank 0 has started: every thread arrives at the cluster's barrier now and
    // waits for its first phase before the remote stores (or, for threads that make none, before the second phase)
    if (cluster_split) cluster_arrive();
    bool cluster_waited = false;

    const int n_items = p.tiles_a * p.tiles_b * p.splits;
    const uint32_t tiles_addr = gt_smem(tiles);

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // The weights do not depend on the kernel before this one: the first stages' weight tiles are
            // asked for at once, while the predecessor still runs, and only the activations wait for it.
            int early = 0;
            if (p.early_w && (int)blockIdx.x < n_items) {
                const int split = blockIdx.x % p.splits, tile = blockIdx.x / p.splits;
                int ta, tb;
                gt_tile_of(tile, p.tiles_a, p.tiles_b, p.group_a, ta, tb);
                const int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.n_kb);
                early = min(STAGES, kb1 - kb0);
                for (int i = 0; i < early; ++i) {
                    mbar_expect_tx(full0 + 8 * i, S::STAGE_BYTES);
                    const uint32_t a_dst = tiles_addr + i * S::STAGE_BYTES;
                    if (p.swap) tma_load_2d(a_dst, &map_a, full0 + 8 * i, (kb0 + i) * GT_BK, ta * GT_BM);
                    else tma_load_2d(a_dst + GT_BM * GT_BK * 2, &map_b, full0 + 8 * i, (kb0 + i) * GT_BK, tb * BN);
                }
            }
            pdl_wait();             // the activations are the predecessor's output
            ACV_TL_MARK(TL_M_WAIT_OVER);
            int s = 0;              // stage of the current k-block, and the parity its "empty" barrier is awaited with
            uint32_t ph = 0;
            for (int item = blockIdx.x; item < n_items && !abort_s; item += gridDim.x) {
                const int split = item % p.splits, tile = item / p.splits;
                int ta, tb;
                gt_tile_of(tile, p.tiles_a, p.tiles_b, p.group_a, ta, tb);
                const int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.n_kb);
                for (int kb = kb0; kb < kb1; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0)) {
                    const uint32_t a_dst = tiles_addr + s * S::STAGE_BYTES;
                    const bool half_done = early > 0;       // this stage's weight tile is already on its way
                    if (half_done) {
                        --early;
                    } else {
                        [[maybe_unused]] const unsigned long long tp0 = ACV_TL_NOW();
                        if (!mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 1); break; }
                        ACV_TL_ADD(TL_M_SUM_FREE_WAIT, tp0);
                        mbar_expect_tx(full0 + 8 * s, S::STAGE_BYTES);
                    }
                    if (kb == p.skip_kb) continue;          // test of the bounded waits: the bytes announced never come
                    [[maybe_unused]] const unsigned long long tp1 = ACV_TL_NOW();
                    if (!(half_done && p.swap)) tma_load_2d(a_dst, &map_a, full0 + 8 * s, kb * GT_BK, ta * GT_BM);
                    if (!(half_done && !p.swap)) tma_load_2d(a_dst + GT_BM * GT_BK * 2, &map_b, full0 + 8 * s, kb * GT_BK, tb * BN);
                    ACV_TL_ADD(TL_M_SUM_LOAD_ISSUE, tp1);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // The one thread's instructions are what a k-block costs beside its products: the descriptors are kept as
            // their low halves (address and leading offset), a stage or 16 elements of k further is one 32-bit add.
            const uint32_t idesc = umma_idesc(BN);
            const uint32_t a_lo0 = umma_desc_lo(tiles_addr), b_lo0 = umma_desc_lo(tiles_addr + GT_BM * GT_BK * 2);
            constexpr uint32_t STAGE_LO = S::STAGE_BYTES >> 4;
            uint32_t local = 0, ph = 0, s_lo = 0;
            int s = 0;
            for (int item = blockIdx.x; item < n_items && !abort_s; item += gridDim.x, ++local) {
                const int split = item % p.splits;
                const int kb0 = split * p.kb_per_split, kb1 = min(kb0 + p.kb_per_split, p.n_kb);
                const uint32_t buf = local & 1, use = local >> 1;
                [[maybe_unused]] const unsigned long long tw0 = ACV_TL_NOW();
                if (!mbar_wait(tempty0 + 8 * buf, (use & 1) ^ 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 2); break; }
                if (p.splits == 1) ACV_TL_ADD(TL_M_SUM_ACC_WAIT, tw0);
                tc_fence_after();
                const uint32_t d = tmem_base + buf * BN;
                bool failed = false;
                for (int kb = kb0; kb < kb1; ++kb) {
                    [[maybe_unused]] const unsigned long long tw1 = ACV_TL_NOW();
                    if (!mbar_wait(full0 + 8 * s, ph, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 3); failed = true; break; }
                    if (p.splits == 1) ACV_TL_ADD(TL_M_SUM_STAGE_WAIT, tw1);
                    if (local == 0 && kb == kb0) ACV_TL_MARK(TL_M_FIRST_FULL);
                    [[maybe_unused]] const unsigned long long ti0 = ACV_TL_NOW();
                    const uint32_t a_lo = a_lo0 + s_lo, b_lo = b_lo0 + s_lo;
                    tc_mma_bf16_h(d, a_lo, b_lo, idesc, kb > kb0 ? 1u : 0u);
#pragma unroll
                    for (int k = 1; k < GT_BK / 16; ++k) tc_mma_bf16_h(d, a_lo + 2 * k, b_lo + 2 * k, idesc, 1u);
                    tc_commit(empty0 + 8 * s);      // frees the stage when these MMAs have read it
                    ACV_TL_ADD(TL_M_SUM_MMA_ISSUE, ti0);
                    ++s; s_lo += STAGE_LO;
                    if (s == STAGES) { s = 0; s_lo = 0; ph ^= 1; }
                }
                if (failed) break;
                tc_commit(tfull0 + 8 * buf);        // the accumulator is complete
                if (item + (int)gridDim.x >= n_items) ACV_TL_MARK(TL_M_LAST_MMA);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5)
        const int wq = warp & 3;                    // the 32 tensor-memory lanes this warp may read
        const int et = threadIdx.x - 64;            // 0..127 among the epilogue threads
        pdl_wait();                                 // results, workspace and counters are shared with earlier kernels
        if (p.qkv && p.swap && (int)blockIdx.x < n_items && (!cluster_split || cluster_ctarank() == 0)) {
            // where each token of the tile stands and goes, and its angles: read now, needed when the tile leaves
            const int tile = blockIdx.x / p.splits;
            int ta0, tb;
            gt_tile_of(tile, p.tiles_a, p.tiles_b, p.group_a, ta0, tb);
            int* pos_s = reinterpret_cast<int*>(aux);
            int* pg_s = pos_s + BN;
            float* cs_s = reinterpret_cast<float*>(pg_s + BN);
            const int D = p.head_dim;
            for (int r = et; r < BN; r += 128) {
                const int t = tb * BN + r;
                int pos = 0, pg = -1;
                if (t < p.M) {
                    pos = p.positions[t];
                    {
                        const int sq = p.seq_of_token[t];
                        pg = p.block_table[(size_t)(p.bt_rows ? p.bt_rows[sq] : sq) * p.bt_stride + pos / p.page_size];
                    }
                    if (pg >= p.num_pages) pg = -1;
                }
                pos_s[r] = pos;
                pg_s[r] = pg;
            }
            if (p.cos_sin) {
                for (int i = et; i < BN * (D >> 2); i += 128) {
                    const int r = i / (D >> 2), c4 = i - r * (D >> 2);
                    const int t = tb * BN + r;
                    int pos = t < p.M ? p.positions[t] : 0;
                    if (pos < 0 || pos >= p.table_rows) pos = 0;
                    reinterpret_cast<float4*>(cs_s)[i] = reinterpret_cast<const float4*>(p.cos_sin + (size_t)pos * D)[c4];
                }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
        uint32_t local = 0;
        for (int item = blockIdx.x; item < n_items && !abort_s; item += gridDim.x, ++local) {
            const int split = item % p.splits, tile = item / p.splits;
            int ta, tb;
            gt_tile_of(tile, p.tiles_a, p.tiles_b, p.group_a, ta, tb);
            const uint32_t buf = local & 1, use = local >> 1;
            if (!mbar_wait(tfull0 + 8 * buf, use & 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 4); break; }
            tc_fence_after();
            [[maybe_unused]] const unsigned long long te0 = ACV_TL_NOW();
            if (et == 0 && item + (int)gridDim.x >= n_items) ACV_TL_MARK(TL_M_ACC_DONE);
            const int row_a = ta * GT_BM + wq * 32 + lane;          // row of the A operand this thread holds
            const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(wq * 32) << 16);
            if (p.splits == 1 && p.qkv && !p.swap) {
                if constexpr (BN == 128 || BN == 256) {
                    if (p.head_dim == 128) gt_store_qkv_rows<BN, 128>(p, taddr, row_a, tb);
                    else gt_store_qkv_rows<BN, 64>(p, taddr, row_a, tb);
                } else if constexpr (BN == 64) {
                    gt_store_qkv_rows<BN, 64>(p, taddr, row_a, tb);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
                if (et == 0) ACV_TL_ADD(TL_M_SUM_EPILOGUE, te0);
                continue;
            }
            if (p.splits == 1) {
                const int rows_b = min(BN, p.RB - tb * BN);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (p.staged && c0 >= rows_b) break;
                    uint32_t r[16];
                    tc_ld16(taddr + c0, r);
                    float v[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r[c]);
                    if (p.staged) gt_stage16(p, tiles, wq * 32 + lane, c0, v, lane);
                    else gt_store16(p, row_a, tb * BN + c0, v, lane);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
                if (et == 0 && !p.swap) ACV_TL_ADD(TL_M_SUM_EPILOGUE, te0);
                if (p.staged) {         // the only item of this CTA: its loads have all been consumed
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (p.qkv) gt_flush_qkv(p, tiles, aux, ta, tb, BN, et);
                    else gt_flush(p, tiles, ta, tb, BN, et);
                }
                continue;
            }
            if (cluster_split) {
                // ---- split K inside a cluster: ranks 1.. put their partial tile into rank 0's shared memory, every store
                // counted at rank 0's barrier; rank 0 waits there for all the bytes and adds the tiles to its own (one
                // item per CTA in this mode)
                const uint32_t rank = cluster_ctarank();
                cluster_wait();
                cluster_waited = true;
                if (rank != 0) {
                    const uint32_t remote = cluster_map(part0, 0) + (rank - 1) * S::PART_BYTES + (wq * 32 + lane) * 4;
                    const uint32_t remote_bar = cluster_map(part_bar, 0);
#pragma unroll 1
                    for (int c0 = 0; c0 < BN; c0 += 16) {
                        uint32_t r[16];
                        tc_ld16(taddr + c0, r);
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            cluster_store_f32_counted(remote + (c0 + c) * (GT_BM * 4), __uint_as_float(r[c]), remote_bar);
                    }
                }
                break;
            }
            // ---- split K: partial tile to the workspace, the CTA that arrives last sums in split order
            float* ws = p.workspace + ((size_t)tile * p.splits + split) * (BN * GT_BM);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t r[16];
                tc_ld16(taddr + c0, r);
#pragma unroll
                for (int c = 0; c < 16; ++c) ws[(c0 + c) * GT_BM + wq * 32 + lane] = __uint_as_float(r[c]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
            __threadfence();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (et == 0) last_s = atomicAdd(&p.counters[tile], 1) == p.splits - 1;
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (last_s) {
                __threadfence();
                const float* wt = p.workspace + (size_t)tile * p.splits * (BN * GT_BM);
                const int rows_b = min(BN, p.RB - tb * BN);
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    if (c0 >= rows_b) break;
                    // sixteen columns at a time: all loads of a split are issued before any store
                    float sum[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) sum[c] = 0.f;
                    for (int sp = 0; sp < p.splits; ++sp) {
                        float v[16];
#pragma unroll
                        for (int c = 0; c < 16; ++c) v[c] = __ldcg(&wt[((size_t)sp * BN + c0 + c) * GT_BM + wq * 32 + lane]);
#pragma unroll
                        for (int c = 0; c < 16; ++c) sum[c] += v[c];
                    }
                    gt_store16(p, row_a, tb * BN + c0, sum, lane);
                }
                if (et == 0) p.counters[tile] = 0;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
        }
    }

    if (cluster_split) {
        if (threadIdx.x == 64) ACV_TL_MARK(TL_M_PART_SENT);
        if (!cluster_waited) cluster_wait();        // every thread that arrived at the cluster's barrier also waits for it
        // Rank 0 waits for the peers' bytes even when its own part has failed: it must not leave (and give its shared
        // memory back) while a peer that knows nothing of that may still be storing into it.
        bool parts_in = true;
        if (warp >= 2 && cluster_ctarank() == 0 && !mbar_wait(part_bar, 0, &never_s, p.wait_limit)) {
            abort_s = 1; atomicExch(p.status, 6); parts_in = false;        // the peers' partial tiles did not all come
        }
        if (threadIdx.x == 64) ACV_TL_MARK(TL_M_CLUSTER_MET);
        if (warp >= 2 && cluster_ctarank() == 0 && !abort_s && parts_in) {
            const int wq = warp & 3;
            const int tile = blockIdx.x / p.splits;
            int ta, tb;
            gt_tile_of(tile, p.tiles_a, p.tiles_b, p.group_a, ta, tb);
            const int row_a = ta * GT_BM + wq * 32 + lane;
            const uint32_t taddr = tmem_base + ((uint32_t)(wq * 32) << 16);
            const float* part = reinterpret_cast<const float*>(tiles + STAGES * S::STAGE_BYTES + 256) + wq * 32 + lane;
            const int rows_b = min(BN, p.RB - tb * BN);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                if (c0 >= rows_b) break;
                uint32_t r[16];
                tc_ld16(taddr + c0, r);
                float sum[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) sum[c] = __uint_as_float(r[c]);
                for (int sp = 1; sp < p.splits; ++sp)           // split order: the sum does not depend on timing
#pragma unroll
                    for (int c = 0; c < 16; ++c) sum[c] += part[((sp - 1) * BN + c0 + c) * GT_BM];
                if (p.staged) gt_stage16(p, tiles, wq * 32 + lane, c0, sum, lane);
                else gt_store16(p, row_a, tb * BN + c0, sum, lane);
            }
            if (p.staged) {
                if (threadIdx.x == 64) ACV_TL_MARK(TL_M_STAGED);
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (p.qkv) gt_flush_qkv(p, tiles, aux, ta, tb, BN, threadIdx.x - 64);
                else gt_flush(p, tiles, ta, tb, BN, threadIdx.x - 64);
            }
        }
    }
    if (threadIdx.x == 64) ACV_TL_MARK(TL_M_STORED);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::TMEM_COLS));
    }
}

// ----------------------------------------------------------------------------- pairs of CTAs on tiles of 256 x 256
// Many tokens (tokens on the rows of A, no split of K): the two CTAs of a cluster of two, on neighbouring SMs, work on
// one tile of 256 tokens by 256 features with tcgen05.mma.cta_group::2.  Each CTA loads its own 128 token rows of A and
// its own 128 of the tile's 256 weight rows of B (32 KB a k-block instead of the 48 KB that a CTA with a tile of its own
// loads, and half of B's shared-memory reads), and holds the accumulator rows of its 128 tokens, all 256 columns, in
// its own tensor memory.  The CTA of rank 0 leads: its "full" barriers count the bytes of both CTAs' loads (the loads
// carry .cta_group::2, which lets a load signal a barrier of the pair's other CTA), its one thread issues the
// products for both, and tcgen05.commit with a multicast mask frees the stage and announces the accumulator in both
// CTAs at once.  The epilogue warps of both CTAs read their own tensor memory and hand the buffer back at the
// leader's barrier (eight arrivals: four warps each).  Warp roles, the two accumulator buffers, the bounded waits
// and the status word are those of gemm_tc_kernel; so are the epilogues (plain, SiLU(gate)*up, q,k,v).
#define GP_BN 256
#define GP_STAGE_BYTES ((GT_BM + GT_BM) * GT_BK * 2)        // a CTA's share of a k-block: 128 rows of A, 128 of B
#define GP_MAX_STAGES 6

__global__ void __launch_bounds__(GT_THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = smem_raw + ((1024u - (gt_smem(smem_raw) & 1023u)) & 1023u);
    const int STAGES = p.stages;
    uint64_t* bars = (uint64_t*)(tiles + STAGES * GP_STAGE_BYTES);
    // bars: full[STAGES] (used in the leader), empty[STAGES], tmem_full[2], tmem_empty[2] (used in the leader)
    const uint32_t full0 = gt_smem(bars), empty0 = full0 + 8 * STAGES;
    const uint32_t tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                // 0 leads the pair
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    ACV_TL(TL_GEMM, 64);
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 8); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {        // the same warp of both CTAs: the pair's tensor memory is given out to both at once
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(&tmem_base_s)), "r"(512));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();     // both CTAs' barriers exist before a load or a commit of the other arrives at them
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();

    const int tiles_a2 = (p.RA + 2 * GT_BM - 1) / (2 * GT_BM);
    const int n_items = tiles_a2 * p.tiles_b;
    const uint32_t tiles_addr = gt_smem(tiles);

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs, each its rows)
        if (lane == 0) {
            const uint32_t lead_full0 = cluster_map(full0, 0);
            int early = 0;              // the first stages' weight rows are asked for while the predecessor still runs
            if (p.early_w && pair < n_items) {
                int ta, tb;
                gt_tile_of(pair, tiles_a2, p.tiles_b, p.group_a, ta, tb);
                early = min(STAGES, p.n_kb);
                for (int i = 0; i < early; ++i) {
                    if (rank == 0) mbar_expect_tx(full0 + 8 * i, 2 * GP_STAGE_BYTES);
                    tma_load_2d_pair(tiles_addr + i * GP_STAGE_BYTES + GT_BM * GT_BK * 2, &map_b, lead_full0 + 8 * i,
                                     i * GT_BK, tb * GP_BN + (int)rank * GT_BM);
                }
            }
            pdl_wait();
            ACV_TL_MARK(TL_M_WAIT_OVER);
            int s = 0;
            uint32_t ph = 0;
            for (int item = pair; item < n_items && !abort_s; item += n_pairs) {
                int ta, tb;
                gt_tile_of(item, tiles_a2, p.tiles_b, p.group_a, ta, tb);
                for (int kb = 0; kb < p.n_kb; ++kb, s = (s + 1 == STAGES ? 0 : s + 1), ph ^= (s == 0)) {
                    const uint32_t a_dst = tiles_addr + s * GP_STAGE_BYTES;
                    const bool half_done = early > 0;
                    if (half_done) {
                        --early;
                    } else {
                        [[maybe_unused]] const unsigned long long tp0 = ACV_TL_NOW();
                        if (!mbar_wait(empty0 + 8 * s, ph ^ 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 1); break; }
                        ACV_TL_ADD(TL_M_SUM_FREE_WAIT, tp0);
                        if (rank == 0) mbar_expect_tx(full0 + 8 * s, 2 * GP_STAGE_BYTES);
                    }
                    if (kb == p.skip_kb) continue;          // test of the bounded waits: the bytes announced never come
                    [[maybe_unused]] const unsigned long long tp1 = ACV_TL_NOW();
                    tma_load_2d_pair(a_dst, &map_a, lead_full0 + 8 * s, kb * GT_BK, ta * 2 * GT_BM + (int)rank * GT_BM);
                    if (!half_done)
                        tma_load_2d_pair(a_dst + GT_BM * GT_BK * 2, &map_b, lead_full0 + 8 * s, kb * GT_BK, tb * GP_BN + (int)rank * GT_BM);
                    ACV_TL_ADD(TL_M_SUM_LOAD_ISSUE, tp1);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (the leader's one thread)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc(GP_BN, 2 * GT_BM);
            const uint32_t a_lo0 = umma_desc_lo(tiles_addr), b_lo0 = umma_desc_lo(tiles_addr + GT_BM * GT_BK * 2);
            constexpr uint32_t STAGE_LO = GP_STAGE_BYTES >> 4;
            uint32_t local = 0, ph = 0, s_lo = 0;
            int s = 0;
            for (int item = pair; item < n_items && !abort_s; item += n_pairs, ++local) {
                const uint32_t buf = local & 1, use = local >> 1;
                [[maybe_unused]] const unsigned long long tw0 = ACV_TL_NOW();
                if (!mbar_wait(tempty0 + 8 * buf, (use & 1) ^ 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 2); break; }
                ACV_TL_ADD(TL_M_SUM_ACC_WAIT, tw0);
                tc_fence_after();
                const uint32_t d = tmem_base + buf * GP_BN;
                bool failed = false;
                for (int kb = 0; kb < p.n_kb; ++kb) {
                    [[maybe_unused]] const unsigned long long tw1 = ACV_TL_NOW();
                    if (!mbar_wait(full0 + 8 * s, ph, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 3); failed = true; break; }
                    ACV_TL_ADD(TL_M_SUM_STAGE_WAIT, tw1);
                    if (local == 0 && kb == 0) ACV_TL_MARK(TL_M_FIRST_FULL);
                    [[maybe_unused]] const unsigned long long ti0 = ACV_TL_NOW();
                    const uint32_t a_lo = a_lo0 + s_lo, b_lo = b_lo0 + s_lo;
                    tc_mma_bf16_pair_h(d, a_lo, b_lo, idesc, kb > 0 ? 1u : 0u);
#pragma unroll
                    for (int k = 1; k < GT_BK / 16; ++k) tc_mma_bf16_pair_h(d, a_lo + 2 * k, b_lo + 2 * k, idesc, 1u);
                    tc_commit_pair(empty0 + 8 * s, 3);      // frees the stage in both CTAs
                    ACV_TL_ADD(TL_M_SUM_MMA_ISSUE, ti0);
                    ++s; s_lo += STAGE_LO;
                    if (s == STAGES) { s = 0; s_lo = 0; ph ^= 1; }
                }
                if (failed) break;
                tc_commit_pair(tfull0 + 8 * buf, 3);        // the accumulator is complete, in both CTAs
                if (item + n_pairs >= n_items) ACV_TL_MARK(TL_M_LAST_MMA);
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
        const int wq = warp & 3;
        pdl_wait();
        const uint32_t lead_tempty0 = cluster_map(tempty0, 0);
        uint32_t local = 0;
        for (int item = pair; item < n_items && !abort_s; item += n_pairs, ++local) {
            int ta, tb;
            gt_tile_of(item, tiles_a2, p.tiles_b, p.group_a, ta, tb);
            const uint32_t buf = local & 1, use = local >> 1;
            if (!mbar_wait(tfull0 + 8 * buf, use & 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 4); break; }
            tc_fence_after();
            [[maybe_unused]] const unsigned long long te0 = ACV_TL_NOW();
            if (threadIdx.x == 64 && item + n_pairs >= n_items) ACV_TL_MARK(TL_M_ACC_DONE);
            const int row_a = ta * 2 * GT_BM + (int)rank * GT_BM + wq * 32 + lane;        // the token this thread holds
            const uint32_t taddr = tmem_base + buf * GP_BN + ((uint32_t)(wq * 32) << 16);
            if (p.qkv) {
                if (p.head_dim == 128) gt_store_qkv_rows<GP_BN, 128>(p, taddr, row_a, tb);
                else gt_store_qkv_rows<GP_BN, 64>(p, taddr, row_a, tb);
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < GP_BN; c0 += 16) {
                    uint32_t r[16];
                    tc_ld16(taddr + c0, r);
                    float v[16];
#pragma unroll
                    for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r[c]);
                    gt_store16(p, row_a, tb * GP_BN + c0, v, lane);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (rank == 0) mbar_arrive(tempty0 + 8 * buf);
                else mbar_arrive_remote(lead_tempty0 + 8 * buf);
            }
            if (threadIdx.x == 64) ACV_TL_ADD(TL_M_SUM_EPILOGUE, te0);
        }
    }
    if (threadIdx.x == 64) ACV_TL_MARK(TL_M_STORED);
    // neither CTA leaves, nor is the pair's tensor memory given back, while the other may still read this one's
    // shared memory or arrive at its barriers
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    }
}

// ----------------------------------------------------------------------------- host side
template <int BN>
static int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, int sm_count, int stages,
                       cudaStream_t stream) {
    using S = GemmShape<BN>;
    if (stages < 2) stages = 2;
    if (stages > S::MAX_STAGES) stages = S::MAX_STAGES;
    // cluster mode needs room for the peers' partial tiles beside the pipeline; else the global workspace serves
    int parts = p.cluster && p.splits > 1 ? p.splits - 1 : 0;
    if (parts && (p.splits > 8 || parts * S::PART_BYTES > 100 * 1024)) { p.cluster = 0; parts = 0; }
    const int aux_bytes = p.qkv && p.swap ? BN * 8 + BN * p.head_dim * 4 : 0;
    while ((parts || aux_bytes) && stages > 2 && S::smem_bytes(stages, parts, aux_bytes) > 226 * 1024) --stages;
    p.stages = stages;
    const int smem = S::smem_bytes(stages, parts, aux_bytes);
    static AcvSmemConfig smem_config;          // per kernel instance and device
    if (int rc = acv_ensure_smem(smem_config, gemm_tc_kernel<BN>, smem)) return rc;
    // CTAs that fit one SM: by shared memory and by tensor-memory columns (512 in all)
    int per_sm = (227 * 1024) / (smem + 1024);
    if (per_sm > 512 / S::TMEM_COLS) per_sm = 512 / S::TMEM_COLS;
    if (per_sm < 1) per_sm = 1;
    if (per_sm > 4) per_sm = 4;
    const long long items = (long long)p.tiles_a * p.tiles_b * p.splits;
    const long long cap = (long long)sm_count * per_sm;
    const int grid = (int)(parts ? items : (items < cap ? items : cap));
    // one item per CTA and rows of C that 16-byte stores can take: the tile leaves through shared memory
    // (the work-space path of split K keeps its direct stores)
    const int esz = p.out_f32 ? 4 : 2;
    p.staged = p.swap && grid == items && (parts || p.splits == 1) && !((uintptr_t)p.C & 15) && !((p.ldc * esz) & 15) &&
               stages * S::STAGE_BYTES >= BN * 128 * esz;
    // the fused q,k,v epilogue exists for staged tiles of up to 32 tokens, and for tokens on M with whole heads in a tile
    if (p.qkv && p.swap && (!p.staged || BN > 32)) return ACV_ERR_SIZE;
    if (p.qkv && !p.swap && (p.splits != 1 || BN < p.head_dim || BN % p.head_dim)) return ACV_ERR_SIZE;
    if (p.qkv && (p.act || p.out_f32)) return ACV_ERR_SIZE;
    acv_launch_cluster(PDL_GEMM, dim3(parts ? p.splits : 1, 1, 1), gemm_tc_kernel<BN>, grid, GT_THREADS, smem, stream, ma, mb, p);
    return acv_launch_status();
}

// Pairs that can be resident at once: clusters of two need two free SMs side by side, which an odd number of SMs in
// a part of the chip does not give; the grid is made of that many pairs and each walks the tiles with that stride.
static int launch_gemm_pair(const CUtensorMap& ma, const CUtensorMap& mb, GemmParams& p, int sm_count, int stages,
                            cudaStream_t stream) {
    if (stages < 2) stages = 2;
    if (stages > GP_MAX_STAGES) stages = GP_MAX_STAGES;
    p.stages = stages;
    const int smem = stages * GP_STAGE_BYTES + 1024 + 256;
    static AcvSmemConfig smem_config;
    if (int rc = acv_ensure_smem(smem_config, gemm_tc_pair_kernel, smem)) return rc;
    static std::mutex mu;
    static int pairs_of_device[64];
    int dev = 0;
    cudaGetDevice(&dev);
    int resident = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64) resident = pairs_of_device[dev];
        if (resident <= 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(2 * (sm_count / 2));
            cfg.blockDim = dim3(GT_THREADS);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&resident, gemm_tc_pair_kernel, &cfg) != cudaSuccess || resident <= 0) {
                cudaGetLastError();
                return ACV_ERR_SIZE;
            }
            if (dev >= 0 && dev < 64) pairs_of_device[dev] = resident;
        }
    }
    if (resident > sm_count / 2) resident = sm_count / 2;
    const long long items = (long long)((p.RA + 2 * GT_BM - 1) / (2 * GT_BM)) * p.tiles_b;
    const int n_pairs = (int)(items < resident ? items : resident);
    if (n_pairs < 1) return ACV_ERR_SIZE;
    p.staged = 0;
    if (p.qkv && (GP_BN < p.head_dim || GP_BN % p.head_dim || p.act || p.out_f32)) return ACV_ERR_SIZE;
    acv_launch_cluster(PDL_GEMM, dim3(2, 1, 1), gemm_tc_pair_kernel, 2 * n_pairs, GT_THREADS, smem, stream, ma, mb, p);
    return acv_launch_status();
}

// Test of the bounded waits, without a fault: the next product launched from this process (and only that one)
// polls each mbarrier at most `wait_limit` times and its producer leaves out the loads of k-block `skip_kb`, so the
// wait for that block runs out, the CTA's roles leave their loops, tensor memory is freed, and `status` holds the
// code of the wait (1 producer, 2 accumulator buffer, 3 operand stage, 4 epilogue).  The output of that launch is
// unspecified; the counters of a split-K workspace may be left non-zero and have to be cleared by the caller.
static unsigned int g_test_wait_limit = 0;
static int g_test_skip_kb = -1;
ACV_API void acv_gemm_tc_test_fault(int wait_limit, int skip_kb) {
    g_test_wait_limit = wait_limit > 0 ? (unsigned int)wait_limit : 0u;
    g_test_skip_kb = skip_kb;
}

// x [M,K] (row stride ldx), w [N,K] (row stride ldw), C [M,N] (row stride ldc) bf16 or float.
// bn: rows of the B operand per tile (16, 32, 64, 128, 160, 192, 224 or 256); swap: the weight is the A operand.
// splits > 1 needs workspace of tiles*splits*bn*128 floats and `tiles` zeroed counters.
// status: one int, 0 unless a bounded wait inside the kernel ran out.
static int gemm_tc_run(GemmParams& p, const void* x, int ldx, const void* w, int ldw, void* C, int ldc, int M, int N, int K,
                       int out_f32, int act, int swap, int bn, int splits, float* workspace, long long workspace_floats,
                       int* counters, long long n_counters, int* status, int sm_count, int stages, int flags,
                       cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || (K % 8) || (ldx % 8) || (ldw % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return ACV_ERR_ALIGN;
    const void* a_ptr = swap ? w : x;
    const void* b_ptr = swap ? x : w;
    p.RA = swap ? N : M;
    p.RB = swap ? M : N;
    p.K = K; p.M = M; p.N = N; p.ldc = ldc; p.swap = swap; p.out_f32 = out_f32; p.act = act; p.cluster = flags & 1; p.early_w = (flags >> 1) & 1;
    if (act && (out_f32 || (N & 1))) return ACV_ERR_SIZE;
    p.tiles_a = (p.RA + GT_BM - 1) / GT_BM;
    p.tiles_b = (p.RB + bn - 1) / bn;
    p.n_kb = (K + GT_BK - 1) / GT_BK;
    // rows of tiles walked together: 2048 tokens' worth where tokens are the rows, all of them where weights are
    p.group_a = swap ? p.tiles_a : ((flags & 4) ? 8 : 16);
    if (splits < 1) splits = 1;
    if (splits > p.n_kb) splits = p.n_kb;
    p.kb_per_split = (p.n_kb + splits - 1) / splits;
    p.splits = (p.n_kb + p.kb_per_split - 1) / p.kb_per_split;
    p.C = C; p.workspace = workspace; p.counters = counters; p.status = status;
    p.wait_limit = g_test_wait_limit ? g_test_wait_limit : GT_WAIT_LIMIT;
    p.skip_kb = g_test_skip_kb;
    g_test_wait_limit = 0; g_test_skip_kb = -1;      // one launch only
    const long long tiles = (long long)p.tiles_a * p.tiles_b;
    if (p.splits > 1 && (tiles * p.splits * bn * GT_BM > workspace_floats || tiles > n_counters)) return ACV_ERR_SCRATCH;
    if (tiles * p.splits > 0x7fffffff) return ACV_ERR_SIZE;
    CUtensorMap ma, mb;
    int rc = make_map(&ma, a_ptr, p.RA, K, swap ? ldw : ldx, GT_BM);
    if (rc) return rc;
    if (flags & 4) {        // pairs of CTAs on tiles of 256 x 256: tokens on rows, no split of K
        if (swap || p.splits != 1 || bn != GP_BN) return ACV_ERR_SIZE;
        rc = make_map(&mb, b_ptr, p.RB, K, ldw, GT_BM);
        if (rc) return rc;
        return launch_gemm_pair(ma, mb, p, sm_count, stages, stream);
    }
    rc = make_map(&mb, b_ptr, p.RB, K, swap ? ldx : ldw, bn);
    if (rc) return rc;
    switch (bn) {
        case 16: return launch_gemm<16>(ma, mb, p, sm_count, stages, stream);
        case 32: return launch_gemm<32>(ma, mb, p, sm_count, stages, stream);
        case 64: return launch_gemm<64>(ma, mb, p, sm_count, stages, stream);
        case 128: return launch_gemm<128>(ma, mb, p, sm_count, stages, stream);
        // widths between 128 and 256 exist for the tokens-on-rows form: with them the number of tiles can be made to
        // fill whole rounds of the SMs (2048 x 4096 in tiles of 128 x 160 is three full rounds of 148, in tiles of
        // 128 x 256 two rounds of which the second is three quarters empty)
        case 160: return launch_gemm<160>(ma, mb, p, sm_count, stages, stream);
        case 192: return launch_gemm<192>(ma, mb, p, sm_count, stages, stream);
        case 224: return launch_gemm<224>(ma, mb, p, sm_count, stages, stream);
        case 256: return launch_gemm<256>(ma, mb, p, sm_count, stages, stream);
        default: return ACV_ERR_SIZE;
    }
}

ACV_TL_EXPORT(gemm_tc)

ACV_API int acv_gemm_tc(const void* x, int ldx, const void* w, int ldw, void* C, int ldc, int M, int N, int K,
                        int out_f32, int act, int swap, int bn, int splits, float* workspace, long long workspace_floats,
                        int* counters, long long n_counters, int* status, int sm_count, int stages, int flags,
                        cudaStream_t stream) {
    GemmParams p;
    p.qkv = 0;
    return gemm_tc_run(p, x, ldx, w, ldw, C, ldc, M, N, K, out_f32, act, swap, bn, splits, workspace, workspace_floats,
                       counters, n_counters, status, sm_count, stages, flags, stream);
}

// The stacked q,k,v projection with its epilogue: C [M, (NH + 2 NKV) D] gets the normed and rotated queries (its
// key and value columns are not written), keys (normed, rotated) and values go to their pages
// [num_pages, NKV, page_size, D] at page block_table[seq][pos / page_size], row pos % page_size; a page index < 0
// writes nothing.  q_w, k_w (float [D]) and cos_sin ([table_rows][D]) may each be null.  Swapped roles with up to 32
// tokens, or tokens on M without a split of K; head size 64 or 128; anything else is refused with ACV_ERR_SIZE.
ACV_API int acv_gemm_tc_qkv(const void* x, int ldx, const void* w, int ldw, void* C, int ldc, int M, int N, int K,
                            int swap, int bn, int splits, float* workspace, long long workspace_floats, int* counters,
                            long long n_counters, int* status, int sm_count, int stages, int flags, int NH, int NKV, int D,
                            const float* q_w, const float* k_w, float eps, const float* cos_sin, int table_rows,
                            const int* positions, const int* seq_of_token, const int* block_table, int bt_stride,
                            const int* bt_rows, void* k_pages, void* v_pages, int page_size, int num_pages, cudaStream_t stream) {
    if ((D != 64 && D != 128) || NH <= 0 || NKV <= 0 || N != (NH + 2 * NKV) * D || (swap && bn > 32) || !k_pages || !v_pages ||
        !positions || !seq_of_token || !block_table || page_size <= 0 || ((uintptr_t)k_pages & 15) || ((uintptr_t)v_pages & 15) ||
        (cos_sin && ((uintptr_t)cos_sin & 15)))
        return ACV_ERR_SIZE;
    GemmParams p;
    p.qkv = 1; p.q_heads = NH; p.kv_heads = NKV; p.head_dim = D; p.q_w = q_w; p.k_w = k_w; p.qk_eps = eps;
    p.cos_sin = cos_sin; p.table_rows = table_rows; p.positions = positions; p.seq_of_token = seq_of_token;
    p.block_table = block_table; p.bt_stride = bt_stride; p.bt_rows = bt_rows; p.k_pages = (bf16*)k_pages; p.v_pages = (bf16*)v_pages;
    p.page_size = page_size; p.num_pages = num_pages;
    return gemm_tc_run(p, x, ldx, w, ldw, C, ldc, M, N, K, 0, 0, swap, bn, splits, workspace, workspace_floats, counters,
                       n_counters, status, sm_count, stages, flags, stream);
}
