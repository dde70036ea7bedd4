// One decoder layer of a decode step (up to 16 requests, one token each) as ONE persistent kernel.
//
// A decode step of a few tokens is bound by the weights it has to stream from memory, and as seven dependent
// launches per layer (norm, q/k/v product, attention, output product, norm, gate/up product, down product) it
// loses a third of its time where one launch hands over to the next: memory idles while a kernel drains, the
// next one starts, asks for its first tiles and waits for them.  Here one CTA per SM runs the whole layer and
// the stream of weight tiles never stops at a phase's end:
//
//   * warp 0 (one thread) is the producer.  It walks ONE sequence of loads for the whole layer - weight tiles of
//     the q/k/v product, key/value tiles of the attention, weight tiles of the output, gate/up and down products -
//     through one ring of shared-memory slots (TMA, mbarriers).  What does not depend on the step (weights; keys
//     and values of earlier tokens) is asked for as soon as a slot is free, however far ahead of the phase that
//     is running; what a phase produces for the next (the activations, the keys and values of this step's token)
//     is asked for once that phase's grid-wide barrier has been passed.  Two cursors walk the same sequence: the
//     leading one issues the independent part of every slot, the trailing one adds the dependent part.
//   * warp 1 (one thread) issues the tcgen05 products of the four matrix products (weights on the tensor core's
//     M side, the tokens are the narrow N = 16 side) into two accumulators in tensor memory.
//   * warps 2..5 do everything else, phase by phase: the two RMS norms (CTA t norms token t), the products'
//     epilogues (split-K partial tiles through a float workspace, summed in split order by the CTA that arrives
//     last at a tile, then SiLU(gate)*up, or per-head norm + rotation + append for q/k/v, or a plain store), and
//     the attention (mma.sync over key tiles that the producer brings, partial results of the splits of a context
//     merged by the CTA that arrives last).
//
// Phases end at grid-wide barriers: counters in global memory at which every CTA arrives once; nobody but the
// consumers of a phase's results waits there.  Every wait in the kernel (mbarrier, grid barrier) is bounded; a wait
// that runs out writes its code into `status`, which also tells every other CTA to give up, and the kernel frees its
// tensor memory and returns.  All 148 CTAs must be resident together: the launcher refuses a grid larger than the
// device's SM count, and a CTA takes a whole SM's shared memory, so CTAs of the kernel before leave before these
// enter.  The arithmetic and the rounding points are those of the separate kernels (elementwise.cu, gemm_tc.cu,
// qk_rope_append.cu, attention_decode.cu), which remain the path for every other batch shape.
#include "gemm_epilogue.cuh"
#include "mma_tiles.cuh"
#include "tensor_map.h"

#define DL_THREADS 192
#define DL_BN 16                                  // tokens (the products' narrow side)
#define DL_SLOT_A (GT_BM * GT_BK * 2)             // a weight tile: 128 features x 64 k = 16 KB
#define DL_SLOT_B (DL_BN * GT_BK * 2)             // an activation tile: 16 tokens x 64 k = 2 KB
#define DL_SLOT (DL_SLOT_A + DL_SLOT_B)           // 18 KB, a multiple of 1024 (the swizzle pattern's anchor)
#define DL_KEYS 32                                // keys of one attention tile (keys and values: 16 KB at D = 128)
#define DL_LOG2E 1.4426950408889634f
#define DL_SCRATCH (33 * 1024)                    // the workers' own memory: norm row / staged tile / attention merge

// grid barriers: phase p is complete when bars[p] == gridDim.x
#define DL_B_NORM1 0
#define DL_B_QKV 1
#define DL_B_ATT 2
#define DL_B_O 3
#define DL_B_NORM2 4
#define DL_B_GU 5
#define DL_B_DONE 6

struct DlGemm {
    GemmParams gp;              // M = tokens, N = features, K, C, ldc, act, qkv ... (swap = 1, staged tiles)
    int tiles, splits, kb_per_split, n_kb, n_items;
    int ctr_base;               // this product's arrival counters start here
    int dep;                    // the grid barrier that its activations wait for
};

struct DlParams {
    int T, H;
    float eps;
    bf16* x;                    // [T, H] the residual stream, updated in place
    const bf16* delta_in;       // [T, H] what the layer before left to be added, or null
    const float* w_norm1;
    const float* w_norm2;
    bf16* h;                    // [T, H] normed activations (both norms)
    bf16* a_out;                // [T, H] the output projection's result (added to x by the second norm)
    DlGemm g[4];                // q/k/v, output, gate/up, down
    // attention
    const bf16* q; int q_stride;            // the q/k/v product's C: queries in its first NH * D columns
    bf16* attn_out; int attn_stride;
    const int* kv_len;
    int NH, NKV, D;
    float scale;
    int att_splits, n_att_items;
    const int* block_table; int bt_stride; const int* bt_rows;
    int page_size, page_shift, num_pages, box_keys;
    float* part_acc; float* part_ml; int* att_counters;
    float* workspace; int* counters;
    unsigned int* bars;
    int* status;
    unsigned int wait_limit;
    int n_slots;
    unsigned long long* trace;  // null, or [gridDim.x][8] device-wide nanosecond stamps of each CTA's phase ends
};

struct DlMaps {
    CUtensorMap w[4];           // the four weights, boxes of 128 rows
    CUtensorMap b[4];           // each product's activations, boxes of 16 rows
    CUtensorMap k, v;           // the cache pages as [pages * kv_heads * page_size, D], boxes of box_keys rows
};

__device__ __forceinline__ unsigned int dl_ld_acquire(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ int dl_ld_status(const int* p) {
    int v;
    asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// one thread: has every CTA arrived at barrier `which`?  (non-blocking)
__device__ __forceinline__ bool dl_passed(const DlParams& p, int which) {
    return dl_ld_acquire(p.bars + which) >= gridDim.x;
}
// one thread: wait for it, bounded.  false: gave up (status written) or another CTA gave up.
__device__ __forceinline__ bool dl_wait_bar(const DlParams& p, int which, volatile int* abort_s, int code) {
    for (unsigned int i = 0; i < p.wait_limit; ++i) {
        if (dl_passed(p, which)) return true;
        if ((i & 63) == 63 && (*abort_s || dl_ld_status(p.status))) { *abort_s = 1; return false; }
        __nanosleep(20);
    }
    *abort_s = 1;
    atomicExch(p.status, code);
    return false;
}

// byte offset of the 16-byte chunk c of row r in a key or value tile as TMA wrote it: atoms of 64 elements
// (128 bytes a row, DL_KEYS rows), chunks of a row exchanged by the 128-byte swizzle
__device__ __forceinline__ int dl_kv_off(int r, int c) {
    return (c >> 3) * (DL_KEYS * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4);
}

// ----------------------------------------------------------------------------- the sequence of ring slots
// Every role walks the same sequence of units (a unit = one slot's load): for each product the k-blocks of this
// CTA's work items, and between the q/k/v and the output product the key tiles of this CTA's attention item.
struct DlSeq {
    int phase;          // 0 q/k/v, 1 attention, 2 output, 3 gate/up, 4 down, 5 end
    int item;           // running index of this CTA's item within the phase
    int kb, kb_end;     // k-block (product) or key tile (attention) and its end
    int tile, split;    // product: the work item's tile and split
    int s;              // slot of the current unit
    unsigned int ph;    // parity of that slot's round
};

struct DlAtt {          // this CTA's attention item
    int active, req, kvh, split, beg, end, p, n_tiles, row;
};

__device__ __forceinline__ int dl_gemm_of(int phase) { return phase == 0 ? 0 : phase - 1; }   // phases 2,3,4 -> products 1,2,3

__device__ __forceinline__ bool dl_seq_enter(const DlParams& p, const DlAtt& att, DlSeq& c) {
    // position on the first unit of (phase, item), moving on through items and phases that hold nothing
    for (;;) {
        if (c.phase >= 5) return false;
        if (c.phase == 1) {
            if (c.item == 0 && att.active && att.n_tiles > 0) { c.kb = 0; c.kb_end = att.n_tiles; return true; }
        } else {
            const DlGemm& g = p.g[dl_gemm_of(c.phase)];
            const int it = blockIdx.x + c.item * gridDim.x;
            if (it < g.n_items) {
                c.split = it % g.splits; c.tile = it / g.splits;
                c.kb = c.split * g.kb_per_split;
                c.kb_end = min(c.kb + g.kb_per_split, g.n_kb);
                if (c.kb < c.kb_end) return true;
                ++c.item;
                continue;
            }
        }
        ++c.phase; c.item = 0;
    }
}
__device__ __forceinline__ bool dl_seq_next(const DlParams& p, const DlAtt& att, DlSeq& c) {
    if (++c.s == p.n_slots) { c.s = 0; c.ph ^= 1; }
    if (++c.kb < c.kb_end) return true;
    ++c.item;
    if (c.phase == 1) { ++c.phase; c.item = 0; }
    return dl_seq_enter(p, att, c);
}

// ----------------------------------------------------------------------------- the kernel
template <int D>
__global__ void __launch_bounds__(DL_THREADS, 1)
decode_layer_kernel(const __grid_constant__ DlMaps maps, const __grid_constant__ DlParams p) {
    constexpr int CH = D / 8, DA = D / 64;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* ring = smem_raw + ((1024u - (gt_smem(smem_raw) & 1023u)) & 1023u);
    const int NS = p.n_slots;
    unsigned char* scratch = ring + NS * DL_SLOT;                       // DL_SCRATCH bytes, the workers'
    unsigned char* aux = scratch + DL_SCRATCH;                          // positions, pages, cos/sin of the tokens
    uint64_t* bars = (uint64_t*)(aux + DL_BN * 8 + DL_BN * D * 4);
    const uint32_t ring_addr = gt_smem(ring);
    const uint32_t full0 = gt_smem(bars), empty0 = full0 + 8 * NS, tfull0 = empty0 + 8 * NS, tempty0 = tfull0 + 16;
    const uint32_t att_done = tempty0 + 16;     // this CTA's workers are through with the key tiles of its attention item
    __shared__ uint32_t tmem_base_s;
    __shared__ volatile int abort_s;
    __shared__ int last_s;
    __shared__ float red_s[4];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < NS; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(tfull0 + 8 * b, 1); mbar_init(tempty0 + 8 * b, 4); }
        mbar_init(att_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(gt_smem(&tmem_base_s)), "r"(32));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    // the ring starts at zero: rows of a key tile that no load fills (beyond the context) are multiplied by a zero
    // probability and must be finite
    for (int i = threadIdx.x; i < NS * DL_SLOT / 16; i += DL_THREADS) reinterpret_cast<uint4*>(ring)[i] = make_uint4(0, 0, 0, 0);
    fence_proxy_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;
    pdl_launch_dependents();

    // ---- this CTA's attention item (the same arithmetic in every role; kv_len is the step's own input, read after
    //      the wait for the kernels before)
    const int n_rep = p.NH / p.NKV;
    auto att_of = [&]() {
        DlAtt a;
        a.active = (int)blockIdx.x < p.n_att_items;
        a.req = a.kvh = a.split = a.beg = a.end = a.p = a.n_tiles = a.row = 0;
        if (a.active) {
            const int pair = blockIdx.x / p.att_splits;
            a.split = blockIdx.x - pair * p.att_splits;
            a.req = pair / p.NKV; a.kvh = pair - a.req * p.NKV;
            a.p = p.kv_len[a.req] - 1;
            const int n_keys = a.p + 1;
            const int chunk = (((n_keys + p.att_splits - 1) / p.att_splits) + 63) & ~63;
            a.beg = a.split * chunk;
            a.end = min(a.beg + chunk, a.p + 1);
            a.n_tiles = a.beg < a.end ? (a.end - a.beg + DL_KEYS - 1) / DL_KEYS : 0;
            a.row = p.bt_rows ? p.bt_rows[a.req] : a.req;
        }
        return a;
    };

    if (warp == 0) {
        // ================================================================== producer
        if (lane == 0) {
            // -- before the step's inputs may be read: weights only.  Fill the ring with the q/k/v product's first tiles.
            DlAtt none; none.active = 0; none.n_tiles = 0;
            DlSeq pre; pre.phase = 0; pre.item = 0; pre.s = 0; pre.ph = 0;
            int early = 0;
            if (dl_seq_enter(p, none, pre) && pre.phase == 0) {
                do {
                    mbar_expect_tx(full0 + 8 * pre.s, DL_SLOT);
                    tma_load_2d(ring_addr + pre.s * DL_SLOT, &maps.w[0], full0 + 8 * pre.s, pre.kb * GT_BK, pre.tile * GT_BM);
                    ++early;
                } while (early < NS && dl_seq_next(p, none, pre) && pre.phase == 0);
            }
            pdl_wait();
            const DlAtt att = att_of();
            const int* bt = p.block_table + (size_t)att.row * p.bt_stride;
            DlSeq lead, trail;          // lead: the independent part of each slot; trail: the dependent part
            lead.phase = 0; lead.item = 0; lead.s = 0; lead.ph = 0;
            trail = lead;
            bool lead_on = dl_seq_enter(p, att, lead), trail_on = dl_seq_enter(p, att, trail);
            unsigned int n_lead = 0, n_trail = 0;       // units that each cursor has passed
            int passed = -1;                            // grid barriers known to be passed: 0 .. passed
            auto dep_of = [&](const DlSeq& c) { return c.phase == 1 ? DL_B_QKV : p.g[dl_gemm_of(c.phase)].dep; };
            // key tile: which of its pages are loaded, and whether it holds this step's own token
            auto att_tile = [&](const DlSeq& c, bool issue) -> uint32_t {
                const int j0 = att.beg + c.kb * DL_KEYS;
                uint32_t bytes = 0;
                for (int j = j0; j < j0 + DL_KEYS && j < att.end; j += p.box_keys) {
                    const int pg = bt[j >> p.page_shift];
                    if (pg < 0 || pg >= p.num_pages) continue;
                    bytes += 2u * DA * p.box_keys * 128u;
                    if (issue) {
                        const uint32_t dst = ring_addr + c.s * DL_SLOT + (j - j0) * 128;
                        const int row = (pg * p.NKV + att.kvh) * p.page_size + (j & (p.page_size - 1));
#pragma unroll
                        for (int a = 0; a < DA; ++a) {
                            tma_load_2d(dst + a * (DL_KEYS * 128), &maps.k, full0 + 8 * c.s, a * 64, row);
                            tma_load_2d(dst + DA * (DL_KEYS * 128) + a * (DL_KEYS * 128), &maps.v, full0 + 8 * c.s, a * 64, row);
                        }
                    }
                }
                return bytes;
            };
            auto holds_new_token = [&](const DlSeq& c) { const int j0 = att.beg + c.kb * DL_KEYS; return att.p >= j0 && att.p < j0 + DL_KEYS; };
            unsigned int spins = 0;
            while (lead_on || trail_on) {
                bool moved = false;
                // -- the leading cursor: every free slot gets its announcement and what does not depend on the step
                while (lead_on) {
                    const bool prefilled = (int)n_lead < early;         // its weight tile is already on its way
                    if (!prefilled && !mbar_try_wait(empty0 + 8 * lead.s, lead.ph ^ 1)) break;
                    if (lead.phase == 1) {
                        const uint32_t bytes = att_tile(lead, false);
                        if (bytes) mbar_expect_tx(full0 + 8 * lead.s, bytes); else mbar_arrive(full0 + 8 * lead.s);
                        if (!holds_new_token(lead)) att_tile(lead, true);
                    } else if (!prefilled) {
                        mbar_expect_tx(full0 + 8 * lead.s, DL_SLOT);
                        tma_load_2d(ring_addr + lead.s * DL_SLOT, &maps.w[dl_gemm_of(lead.phase)], full0 + 8 * lead.s,
                                    lead.kb * GT_BK, lead.tile * GT_BM);
                    }
                    ++n_lead;
                    lead_on = dl_seq_next(p, att, lead);
                    moved = true;
                }
                // -- the trailing cursor: dependent loads of the units that the leading one has opened, as far as the
                //    grid barriers that they wait for have been passed (one look at a barrier per turn)
                while (trail_on && n_trail < n_lead) {
                    const int dep = dep_of(trail);
                    if (dep > passed) {
                        if (!dl_passed(p, dep)) break;
                        passed = dep;
                        asm volatile("fence.proxy.async.global;" ::: "memory");
                    }
                    if (trail.phase == 1) {
                        if (holds_new_token(trail)) att_tile(trail, true);
                    } else {
                        tma_load_2d(ring_addr + trail.s * DL_SLOT + DL_SLOT_A, &maps.b[dl_gemm_of(trail.phase)],
                                    full0 + 8 * trail.s, trail.kb * GT_BK, 0);
                    }
                    ++n_trail;
                    trail_on = dl_seq_next(p, att, trail);
                    moved = true;
                }
                if (moved) { spins = 0; continue; }
                if (++spins > p.wait_limit) { abort_s = 1; atomicExch(p.status, 21); break; }
                if ((spins & 63) == 63 && (abort_s || dl_ld_status(p.status))) { abort_s = 1; break; }
            }
        }
    } else if (warp == 1) {
        // ================================================================== MMA issuer
        if (lane == 0) {
            pdl_wait();
            const DlAtt att = att_of();
            const uint32_t idesc = umma_idesc(DL_BN);
            DlSeq c; c.phase = 0; c.item = 0; c.s = 0; c.ph = 0;
            bool on = dl_seq_enter(p, att, c);
            uint32_t local = 0;
            bool past_attention = false;
            while (on && !abort_s) {
                if (c.phase == 1) { on = dl_seq_next(p, att, c); continue; }        // key tiles are the workers'
                // A wait on a slot tells its rounds apart by one bit.  The slots of the output product's first tiles
                // held key tiles a round before: this thread may look at them only when the workers are through with
                // the key tiles, or it would take a key tile that has not landed yet for its own tile of weights.
                if (c.phase >= 2 && !past_attention) {
                    if (!mbar_wait(att_done, 0, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 27); break; }
                    past_attention = true;
                }
                const uint32_t buf = local & 1, use = local >> 1;
                if (!mbar_wait(tempty0 + 8 * buf, (use & 1) ^ 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 22); break; }
                tc_fence_after();
                const uint32_t d = tmem_base + buf * DL_BN;
                const int phase = c.phase, item = c.item, kb0 = c.kb;
                bool failed = false;
                while (on && c.phase == phase && c.item == item) {
                    if (!mbar_wait(full0 + 8 * c.s, c.ph, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 23); failed = true; break; }
                    tc_fence_after();
                    const uint32_t a_addr = ring_addr + c.s * DL_SLOT, b_addr = a_addr + DL_SLOT_A;
#pragma unroll
                    for (int k = 0; k < GT_BK / 16; ++k)
                        tc_mma_bf16(d, umma_desc(a_addr + k * 32), umma_desc(b_addr + k * 32), idesc, (c.kb > kb0 || k > 0) ? 1u : 0u);
                    tc_commit(empty0 + 8 * c.s);
                    on = dl_seq_next(p, att, c);
                }
                if (failed) break;
                tc_commit(tfull0 + 8 * buf);
                ++local;
            }
        }
    } else {
        // ================================================================== workers (warps 2..5)
        const int wq = warp & 3;                    // the tensor-memory lanes this warp may read
        const int et = threadIdx.x - 64;            // 0..127
        const int wr = warp - 2;                    // 0..3: the warp's rank among the workers
        pdl_wait();
        const DlAtt att = att_of();
        const int T = p.T, H = p.H;
        auto sync_workers = [&]() { asm volatile("bar.sync 1, 128;" ::: "memory"); };
        auto stamp = [&](int i) {
            if (p.trace && et == 0) {
                unsigned long long t;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
                p.trace[(size_t)blockIdx.x * 8 + i] = t;
            }
        };
        auto arrive = [&](int which) {              // this CTA's part of a phase is written
            __threadfence();
            sync_workers();
            if (et == 0) atomicAdd(p.bars + which, 1u);
            stamp(which + 1);
        };
        auto wait_bar = [&](int which, int code) -> bool {      // all workers wait for a grid barrier
            if (et == 0) last_s = dl_wait_bar(p, which, &abort_s, code) ? 1 : 0;
            sync_workers();
            const bool ok = last_s != 0;
            sync_workers();
            return ok;
        };
        // -- where each token stands and goes, and its angles (for the q/k/v epilogue)
        {
            int* pos_s = reinterpret_cast<int*>(aux);
            int* pg_s = pos_s + DL_BN;
            float* cs_s = reinterpret_cast<float*>(pg_s + DL_BN);
            const GemmParams& q = p.g[0].gp;
            for (int r = et; r < DL_BN; r += 128) {
                int pos = 0, pg = -1;
                if (r < T) {
                    pos = q.positions[r];
                    const int sq = q.seq_of_token[r];
                    pg = q.block_table[(size_t)(q.bt_rows ? q.bt_rows[sq] : sq) * q.bt_stride + pos / q.page_size];
                    if (pg >= q.num_pages) pg = -1;
                }
                pos_s[r] = pos; pg_s[r] = pg;
            }
            if (q.cos_sin) {
                for (int i = et; i < DL_BN * (D >> 2); i += 128) {
                    const int r = i / (D >> 2), c4 = i - r * (D >> 2);
                    int pos = r < T ? q.positions[r] : 0;
                    if (pos < 0 || pos >= q.table_rows) pos = 0;
                    reinterpret_cast<float4*>(cs_s)[i] = reinterpret_cast<const float4*>(q.cos_sin + (size_t)pos * D)[c4];
                }
            }
            sync_workers();
        }

        // -- x += delta; h = rmsnorm(x) * w for token `blockIdx.x` (add_rmsnorm_vec_kernel's arithmetic)
        auto norm_row = [&](const bf16* delta, const float* w) {
            const int t = blockIdx.x;
            float* row = reinterpret_cast<float*>(scratch);
            uint4* xr = reinterpret_cast<uint4*>(p.x + (size_t)t * H);
            const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + (size_t)t * H) : nullptr;
            float ss = 0.f;
            for (int c = et; c < H / 8; c += 128) {
                uint4 xa = xr[c];
                const bf16* xe = reinterpret_cast<const bf16*>(&xa);
                float v[8];
                if (dr) {
                    uint4 da = dr[c];
                    const bf16* de = reinterpret_cast<const bf16*>(&da);
                    bf16 summed[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) { summed[e] = __float2bfloat16_rn(__bfloat162float(xe[e]) + __bfloat162float(de[e])); v[e] = __bfloat162float(summed[e]); }
                    xr[c] = *reinterpret_cast<const uint4*>(summed);
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = __bfloat162float(xe[e]);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) { row[c * 8 + e] = v[e]; ss += v[e] * v[e]; }
            }
            ss = warp_sum(ss);
            if (lane == 0) red_s[wr] = ss;
            sync_workers();
            ss = red_s[0] + red_s[1] + red_s[2] + red_s[3];
            const float rs = rsqrtf(ss / (float)H + p.eps);
            uint4* o = reinterpret_cast<uint4*>(p.h + (size_t)t * H);
            for (int c = et; c < H / 8; c += 128) {
                bf16 res[8];
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    res[e] = __float2bfloat16_rn(__bfloat162float(__float2bfloat16_rn(row[c * 8 + e] * rs)) * w[c * 8 + e]);
                o[c] = *reinterpret_cast<const uint4*>(res);
            }
            sync_workers();
        };

        // -- the epilogues of one product's work items
        uint32_t local = 0;
        auto gemm_items = [&](int gi) -> bool {
            const DlGemm& g = p.g[gi];
            for (int it = blockIdx.x; it < g.n_items && !abort_s; it += gridDim.x) {
                const int split = it % g.splits, tile = it / g.splits;
                if (split * g.kb_per_split >= g.n_kb) continue;
                const uint32_t buf = local & 1, use = local >> 1;
                ++local;
                if (!mbar_wait(tfull0 + 8 * buf, use & 1, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 24); return false; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + buf * DL_BN + ((uint32_t)(wq * 32) << 16);
                const int f = wq * 32 + lane;                       // the feature of the tile that this thread holds
                float v[16];
                {
                    uint32_t r[16];
                    tc_ld16(taddr, r);
#pragma unroll
                    for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(r[c]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tempty0 + 8 * buf);
                bool finish = true;
                if (g.splits > 1) {
                    float* ws = p.workspace + ((size_t)tile * g.splits + split) * (DL_BN * GT_BM);
#pragma unroll
                    for (int c = 0; c < 16; ++c) ws[c * GT_BM + f] = v[c];
                    __threadfence();
                    sync_workers();
                    if (et == 0) last_s = atomicAdd(&p.counters[g.ctr_base + tile], 1) == g.splits - 1;
                    sync_workers();
                    finish = last_s != 0;
                    if (finish) {
                        __threadfence();
                        const float* wt = p.workspace + (size_t)tile * g.splits * (DL_BN * GT_BM);
#pragma unroll
                        for (int c = 0; c < 16; ++c) v[c] = 0.f;
                        for (int sp = 0; sp < g.splits; ++sp) {         // split order: the sum does not depend on timing
                            float w16[16];
#pragma unroll
                            for (int c = 0; c < 16; ++c) w16[c] = __ldcg(&wt[((size_t)sp * DL_BN + c) * GT_BM + f]);
#pragma unroll
                            for (int c = 0; c < 16; ++c) v[c] += w16[c];
                        }
                        if (et == 0) p.counters[g.ctr_base + tile] = 0;
                    }
                    sync_workers();
                }
                if (finish) {
                    gt_stage16(g.gp, scratch, f, 0, v, lane);
                    sync_workers();
                    if (g.gp.qkv) gt_flush_qkv(g.gp, scratch, aux, tile, 0, DL_BN, et);
                    else gt_flush(g.gp, scratch, tile, 0, DL_BN, et);
                    sync_workers();
                }
            }
            return !abort_s;
        };

        // -- attention of this CTA's (request, kv-head, split): attention_decode.cu's arithmetic on tiles of 32 keys
        auto attention = [&](int unit0) {
            unsigned char* q_s = scratch;                                       // [16][D], read into registers at once
            float* wm = reinterpret_cast<float*>(scratch);                      // afterwards: [4][16] maxima
            float* wl = wm + 64;                                                // [4][16] sums
            float* wacc = wl + 64;                                              // [4][16][D]
            const int tok = att.req;                                            // one token per request, in order
            for (int id = et; id < 16 * CH; id += 128) {
                const int r = id / CH, c = id % CH;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (r < n_rep) v = *reinterpret_cast<const uint4*>(p.q + (size_t)tok * p.q_stride + (size_t)(att.kvh * n_rep + r) * D + c * 8);
                *reinterpret_cast<uint4*>(q_s + tile_off<D>(r, c)) = v;
            }
            sync_workers();
            uint32_t qf[D / 16][4];
            {
                const int mi = lane >> 3, r = lane & 7;
#pragma unroll
                for (int kd = 0; kd < D / 16; ++kd)
                    ldmatrix_x4(qf[kd], smem_u32(q_s + tile_off<D>((mi & 1) * 8 + r, kd * 2 + (mi >> 1))));
            }
            float acc[D / 8][4];
#pragma unroll
            for (int i = 0; i < D / 8; ++i)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[i][e] = 0.f;
            float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
            const float scale_log2 = p.scale * DL_LOG2E;
            const int mi = lane >> 3, lr = lane & 7;
            bool ok = true;
            // Four tiles at a time, one to a warp, and the warps meet after each four: a wait on a slot's barrier tells
            // the phases apart by one bit, so no warp may come to a slot a whole round of the ring before the warp that
            // had the slot's tile of the round before (the ring holds more than four slots).
            for (int i0 = 0; i0 < att.n_tiles; i0 += 4, sync_workers()) {
                const int i = i0 + wr;
                if (i >= att.n_tiles || !ok) continue;
                const int n = unit0 + i;
                const int s = n % NS;
                const uint32_t ph = (uint32_t)(n / NS) & 1u;
                if (!mbar_wait(full0 + 8 * s, ph, &abort_s, p.wait_limit)) { abort_s = 1; atomicExch(p.status, 25); ok = false; continue; }
                const uint32_t kbase = ring_addr + s * DL_SLOT, vbase = kbase + DA * (DL_KEYS * 128);
#pragma unroll
                for (int half = 0; half < DL_KEYS / 16; ++half) {
                    const int jw = att.beg + i * DL_KEYS + half * 16;      // first key of these 16
                    if (jw >= att.end) break;
                    float sc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
                    for (int kd = 0; kd < D / 16; ++kd) {
                        uint32_t b[4];
                        ldmatrix_x4(b, kbase + dl_kv_off(half * 16 + (mi >> 1) * 8 + lr, kd * 2 + (mi & 1)));
                        mma_bf16(sc[0], qf[kd], b[0], b[1]);
                        mma_bf16(sc[1], qf[kd], b[2], b[3]);
                    }
                    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = jw + nt * 8 + (lane & 3) * 2 + (e & 1);
                            const float v = j < att.end ? sc[nt][e] * scale_log2 : -INFINITY;
                            sc[nt][e] = v;
                            mx[e >> 1] = fmaxf(mx[e >> 1], v);
                        }
                    float alpha[2], m_use[2];
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 1));
                        mx[hh] = fmaxf(mx[hh], __shfl_xor_sync(0xffffffffu, mx[hh], 2));
                        const float m_new = fmaxf(m_run[hh], mx[hh]);
                        m_use[hh] = m_new == -INFINITY ? 0.f : m_new;
                        alpha[hh] = exp2f(m_run[hh] - m_use[hh]);
                        m_run[hh] = m_new;
                        l_run[hh] *= alpha[hh];
                    }
                    uint32_t pa[4];
                    float pv[2][4];
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            pv[nt][e] = exp2f(sc[nt][e] - m_use[e >> 1]);
                            l_run[e >> 1] += pv[nt][e];
                        }
                    pa[0] = pack_bf16(pv[0][0], pv[0][1]);
                    pa[1] = pack_bf16(pv[0][2], pv[0][3]);
                    pa[2] = pack_bf16(pv[1][0], pv[1][1]);
                    pa[3] = pack_bf16(pv[1][2], pv[1][3]);
                    if (alpha[0] != 1.f || alpha[1] != 1.f) {
#pragma unroll
                        for (int ii = 0; ii < D / 8; ++ii) {
                            acc[ii][0] *= alpha[0]; acc[ii][1] *= alpha[0];
                            acc[ii][2] *= alpha[1]; acc[ii][3] *= alpha[1];
                        }
                    }
#pragma unroll
                    for (int nd = 0; nd < D / 16; ++nd) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, vbase + dl_kv_off(half * 16 + (mi & 1) * 8 + lr, nd * 2 + (mi >> 1)));
                        mma_bf16(acc[2 * nd], pa, b[0], b[1]);
                        mma_bf16(acc[2 * nd + 1], pa, b[2], b[3]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * s);        // the slot may take its next load
            }
            sync_workers();
            // ---- merge the four warps (q_s is no longer needed: its place takes the partial results)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 1);
                l_run[hh] += __shfl_xor_sync(0xffffffffu, l_run[hh], 2);
            }
            {
                const int r0 = lane >> 2, c0 = (lane & 3) * 2;
                if ((lane & 3) == 0) {
                    wm[wr * 16 + r0] = m_run[0]; wm[wr * 16 + r0 + 8] = m_run[1];
                    wl[wr * 16 + r0] = l_run[0]; wl[wr * 16 + r0 + 8] = l_run[1];
                }
#pragma unroll
                for (int i = 0; i < D / 8; ++i) {
                    float* a0 = wacc + ((wr * 16 + r0) * D) + i * 8 + c0;
                    float* a1 = wacc + ((wr * 16 + r0 + 8) * D) + i * 8 + c0;
                    a0[0] = acc[i][0]; a0[1] = acc[i][1];
                    a1[0] = acc[i][2]; a1[1] = acc[i][3];
                }
            }
            sync_workers();
            const int n_splits = p.att_splits;
            const int pair = att.req * p.NKV + att.kvh;
            const size_t part = (size_t)pair * n_splits + att.split;
            for (int idx = et; idx < n_rep * D; idx += 128) {
                const int r = idx / D, d = idx % D;
                float M = -INFINITY;
#pragma unroll
                for (int w = 0; w < 4; ++w) M = fmaxf(M, wm[w * 16 + r]);
                float L = 0.f, O = 0.f;
                if (M != -INFINITY) {
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const float fsc = exp2f(wm[w * 16 + r] - M);
                        L += wl[w * 16 + r] * fsc;
                        O += wacc[(w * 16 + r) * D + d] * fsc;
                    }
                }
                if (n_splits == 1) {
                    p.attn_out[(size_t)tok * p.attn_stride + (size_t)(att.kvh * n_rep + r) * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
                } else {
                    p.part_acc[(part * n_rep + r) * D + d] = O;
                    if (d == 0) {
                        p.part_ml[(part * n_rep + r) * 2] = M;
                        p.part_ml[(part * n_rep + r) * 2 + 1] = L;
                    }
                }
            }
            if (n_splits == 1) { sync_workers(); return; }
            __threadfence();
            sync_workers();
            if (et == 0) last_s = atomicAdd(&p.att_counters[pair], 1) == n_splits - 1;
            sync_workers();
            const bool last = last_s != 0;
            sync_workers();
            if (!last) return;
            __threadfence();
            const size_t base = (size_t)pair * n_splits;
            for (int idx = et; idx < n_rep * D; idx += 128) {
                const int r = idx / D, d = idx % D;
                float M = -INFINITY;
                for (int sp = 0; sp < n_splits; ++sp) M = fmaxf(M, __ldcg(&p.part_ml[((base + sp) * n_rep + r) * 2]));
                float L = 0.f, O = 0.f;
                if (M != -INFINITY) {
                    for (int sp = 0; sp < n_splits; ++sp) {         // split order
                        const float fsc = exp2f(__ldcg(&p.part_ml[((base + sp) * n_rep + r) * 2]) - M);
                        L += __ldcg(&p.part_ml[((base + sp) * n_rep + r) * 2 + 1]) * fsc;
                        O += __ldcg(&p.part_acc[((base + sp) * n_rep + r) * D + d]) * fsc;
                    }
                }
                p.attn_out[(size_t)tok * p.attn_stride + (size_t)(att.kvh * n_rep + r) * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
            }
            if (et == 0) p.att_counters[pair] = 0;
        };

        // ---- the layer, phase by phase
        bool ok = true;
        stamp(0);
        if ((int)blockIdx.x < T) norm_row(p.delta_in, p.w_norm1);
        arrive(DL_B_NORM1);
        // units of this CTA's q/k/v items: where its key tiles start in the sequence of slots
        int unit0 = 0;
        for (int it = blockIdx.x; it < p.g[0].n_items; it += gridDim.x) {
            const int split = it % p.g[0].splits;
            const int kb0 = split * p.g[0].kb_per_split;
            unit0 += max(0, min(kb0 + p.g[0].kb_per_split, p.g[0].n_kb) - kb0);
        }
        ok = gemm_items(0);
        arrive(DL_B_QKV);
        if (ok && att.active) {
            ok = wait_bar(DL_B_QKV, 31);
            if (ok) attention(unit0);
        }
        if (et == 0) mbar_arrive(att_done);
        arrive(DL_B_ATT);
        if (ok) ok = gemm_items(1);
        arrive(DL_B_O);
        if (ok && (int)blockIdx.x < T) {
            ok = wait_bar(DL_B_O, 32);
            if (ok) norm_row(p.a_out, p.w_norm2);
        }
        arrive(DL_B_NORM2);
        if (ok) ok = gemm_items(2);
        arrive(DL_B_GU);
        if (ok) gemm_items(3);
        __threadfence();
        stamp(7);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32));
    }
    // the CTA that leaves last puts the grid barriers back to zero for the next launch
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(p.bars + DL_B_DONE, 1u) == gridDim.x - 1) {
            for (int i = 0; i <= DL_B_DONE; ++i) p.bars[i] = 0;
            __threadfence();
        }
    }
}

// ----------------------------------------------------------------------------- host side
static int dl_pick_splits(int tiles, int n_kb, int grid) {
    int best = 1;
    long long best_cost = -1;
    for (int s = 1; s <= 16 && s <= n_kb; ++s) {
        const int kbps = (n_kb + s - 1) / s;
        const int real = (n_kb + kbps - 1) / kbps;
        const long long rounds = ((long long)tiles * real + grid - 1) / grid;
        // a work item's epilogue (partial tile out, arrival, the last one's sum) hides behind the next item's loads
        // only when the item streams long enough: count an item as at least 8 k-blocks; then fewer partial tiles
        const long long cost = rounds * (kbps > 8 ? kbps : 8) * 32 + real;
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = real; }
    }
    return best;
}

struct DlLayerArgs {
    // sizes
    int T, H, I, NH, NKV, D;
    float eps, qk_eps, scale;
    // tensors (device pointers)
    void* x; const void* delta_in; const float* w_norm1; const float* w_norm2;
    const void* w_qkv; const void* w_o; const void* w_gu; const void* w_down;
    const float* q_norm; const float* k_norm; const float* cos_sin; int table_rows;
    const int* positions; const int* seq_of_token; const int* kv_len;
    const int* block_table; int bt_stride; const int* bt_rows;
    void* k_pages; void* v_pages; int page_size, num_pages;
    // activations of the layer (device scratch, [16 rows] each) and its result
    void* h; void* qkv; void* attn_out; void* a_out; void* act; void* delta_out;
    // scratch: workspace floats, counters ints (zero), attention partials, barriers (8 zeroed uints), status
    float* workspace; long long workspace_floats; int* counters; long long n_counters;
    float* part; long long part_floats; int* att_counters; long long n_att_counters;   // partial results of the attention's splits
    unsigned int* bars; int* status;
    int sm_count; int max_kv;
    unsigned long long* trace;      // optional: [sm_count][8] time stamps (see DlParams)
};

// Whether the fused kernel takes a layer of these sizes (the separate kernels take everything else).
ACV_API int acv_decode_layer_takes(int T, int H, int I, int NH, int NKV, int D, int page_size, int window) {
    if (T < 1 || T > DL_BN || window > 0) return 0;
    if (D != 64 && D != 128) return 0;
    if (NKV <= 0 || NH % NKV || NH / NKV > 16) return 0;
    if (H % 64 || I % 64 || H > 8192) return 0;
    if (page_size < 16 || (page_size & (page_size - 1))) return 0;
    return 1;
}

template <int D>
static int dl_launch(const DlMaps& maps, const DlParams& p, int grid, int smem, cudaStream_t stream) {
    static AcvSmemConfig smem_config;
    if (int rc = acv_ensure_smem(smem_config, decode_layer_kernel<D>, smem)) return rc;
    acv_launch(PDL_GEMM, decode_layer_kernel<D>, dim3(grid), dim3(DL_THREADS), (size_t)smem, stream, maps, p);
    return acv_launch_status();
}

ACV_API int acv_decode_layer(const DlLayerArgs* a, cudaStream_t stream) {
    if (!acv_decode_layer_takes(a->T, a->H, a->I, a->NH, a->NKV, a->D, a->page_size, 0)) return ACV_ERR_SIZE;
    const int grid = a->sm_count;
    if (grid < DL_BN) return ACV_ERR_SIZE;
    int max_sms = 0, dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&max_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return ACV_ERR_SIZE;
    if (grid > max_sms) return ACV_ERR_SIZE;          // every CTA has to be resident: one per SM at most
    DlParams p;
    DlMaps maps;
    const int T = a->T, H = a->H, D = a->D, NH = a->NH, NKV = a->NKV;
    const int q_size = NH * D, kv_size = NKV * D;
    p.T = T; p.H = H; p.eps = a->eps;
    p.x = (bf16*)a->x; p.delta_in = (const bf16*)a->delta_in; p.w_norm1 = a->w_norm1; p.w_norm2 = a->w_norm2;
    p.h = (bf16*)a->h; p.a_out = (bf16*)a->a_out;
    // the four products: N, K, weights, activations in, result out
    const int Ns[4] = {q_size + 2 * kv_size, H, 2 * a->I, H};
    const int Ks[4] = {H, q_size, H, a->I};
    const void* Ws[4] = {a->w_qkv, a->w_o, a->w_gu, a->w_down};
    const void* Bs[4] = {a->h, a->attn_out, a->h, a->act};
    void* Cs[4] = {a->qkv, a->a_out, a->act, a->delta_out};
    const int ldcs[4] = {q_size + 2 * kv_size, H, a->I, H};
    const int deps[4] = {DL_B_NORM1, DL_B_ATT, DL_B_NORM2, DL_B_GU};
    int ctr = 0;
    long long ws_need = 0;
    for (int i = 0; i < 4; ++i) {
        DlGemm& g = p.g[i];
        GemmParams& gp = g.gp;
        if (Ks[i] % 8 || ((uintptr_t)Ws[i] & 15) || ((uintptr_t)Bs[i] & 15) || ((uintptr_t)Cs[i] & 15) || (ldcs[i] % 8)) return ACV_ERR_ALIGN;
        gp.RA = Ns[i]; gp.RB = T; gp.K = Ks[i]; gp.M = T; gp.N = Ns[i]; gp.ldc = ldcs[i]; gp.swap = 1; gp.out_f32 = 0;
        gp.act = i == 2 ? 1 : 0; gp.qkv = i == 0 ? 1 : 0; gp.staged = 1; gp.cluster = 0; gp.early_w = 1;
        gp.C = Cs[i]; gp.workspace = a->workspace; gp.counters = a->counters; gp.status = a->status;
        gp.wait_limit = GT_WAIT_LIMIT; gp.skip_kb = -1;
        gp.q_heads = NH; gp.kv_heads = NKV; gp.head_dim = D; gp.q_w = a->q_norm; gp.k_w = a->k_norm; gp.qk_eps = a->qk_eps;
        gp.cos_sin = a->cos_sin; gp.table_rows = a->table_rows; gp.positions = a->positions; gp.seq_of_token = a->seq_of_token;
        gp.block_table = a->block_table; gp.bt_stride = a->bt_stride; gp.bt_rows = a->bt_rows;
        gp.k_pages = (bf16*)a->k_pages; gp.v_pages = (bf16*)a->v_pages; gp.page_size = a->page_size; gp.num_pages = a->num_pages;
        g.tiles = (Ns[i] + GT_BM - 1) / GT_BM;
        g.n_kb = (Ks[i] + GT_BK - 1) / GT_BK;
        gp.tiles_a = g.tiles; gp.tiles_b = 1; gp.n_kb = g.n_kb;
        const int s = dl_pick_splits(g.tiles, g.n_kb, grid);
        g.kb_per_split = (g.n_kb + s - 1) / s;
        g.splits = (g.n_kb + g.kb_per_split - 1) / g.kb_per_split;
        gp.splits = g.splits; gp.kb_per_split = g.kb_per_split;
        g.n_items = g.tiles * g.splits;
        g.ctr_base = ctr;
        ctr += g.tiles;
        g.dep = deps[i];
        if (g.splits > 1 && (long long)g.tiles * g.splits * DL_BN * GT_BM > ws_need) ws_need = (long long)g.tiles * g.splits * DL_BN * GT_BM;
        int rc = make_map(&maps.w[i], Ws[i], Ns[i], Ks[i], Ks[i], GT_BM);
        if (rc) return rc;
        rc = make_map(&maps.b[i], Bs[i], T, Ks[i], Ks[i], DL_BN);
        if (rc) return rc;
    }
    if (ws_need > a->workspace_floats || ctr > a->n_counters) return ACV_ERR_SCRATCH;
    // attention: the splits of every (request, kv-head) pair, one work item per CTA
    const int pairs = T * NKV;
    if (pairs > grid) return ACV_ERR_SIZE;
    int splits = grid / pairs;
    const int by_len = (a->max_kv + 127) / 128;
    if (splits > by_len) splits = by_len;
    if (splits < 1) splits = 1;
    p.att_splits = splits; p.n_att_items = pairs * splits;
    const long long n_rep = NH / NKV;
    if (splits > 1 && ((long long)p.n_att_items * n_rep * (D + 2) > a->part_floats || pairs > a->n_att_counters)) return ACV_ERR_SCRATCH;
    p.q = (const bf16*)a->qkv; p.q_stride = q_size + 2 * kv_size; p.attn_out = (bf16*)a->attn_out; p.attn_stride = q_size;
    p.kv_len = a->kv_len; p.NH = NH; p.NKV = NKV; p.D = D; p.scale = a->scale;
    p.block_table = a->block_table; p.bt_stride = a->bt_stride; p.bt_rows = a->bt_rows;
    p.page_size = a->page_size; p.num_pages = a->num_pages;
    p.page_shift = 0;
    while ((1 << p.page_shift) < a->page_size) ++p.page_shift;
    p.box_keys = a->page_size < DL_KEYS ? a->page_size : DL_KEYS;
    p.part_acc = a->part; p.part_ml = a->part + (long long)p.n_att_items * n_rep * D; p.att_counters = a->att_counters;
    p.workspace = a->workspace; p.counters = a->counters; p.bars = a->bars; p.status = a->status;
    p.wait_limit = GT_WAIT_LIMIT;
    p.trace = a->trace;
    const long long pool_rows = (long long)a->num_pages * NKV * a->page_size;
    if (pool_rows > 0x7fffffffLL || ((uintptr_t)a->k_pages & 15) || ((uintptr_t)a->v_pages & 15)) return ACV_ERR_SIZE;
    int rc = make_map(&maps.k, a->k_pages, pool_rows, D, D, p.box_keys);
    if (rc) return rc;
    rc = make_map(&maps.v, a->v_pages, pool_rows, D, D, p.box_keys);
    if (rc) return rc;
    // shared memory: as many slots as fit beside the workers' own memory
    const int fixed = 1024 + DL_SCRATCH + DL_BN * 8 + DL_BN * D * 4 + 512;
    int slots = (227 * 1024 - fixed) / DL_SLOT;
    if (slots > 12) slots = 12;
    if (slots < 4) return ACV_ERR_SIZE;
    p.n_slots = slots;
    const int smem = fixed + slots * DL_SLOT;
    if (D == 64) return dl_launch<64>(maps, p, grid, smem, stream);
    return dl_launch<128>(maps, p, grid, smem, stream);
}
