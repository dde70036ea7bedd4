"""The hot kernels one by one: ``acvram bench --what kernels`` (the reference's name for its per-kernel
measurements, acvram/cli.py:1476), and the small cases that are profiled under ncu.

    acvram bench --what kernels [--case NAME] [--json]
    python -m acvram_b200.profile_cases gemm_decode|gemm_prefill|attention_decode|attention_prefill [--reps N]

Each case runs a few launches of one kernel at the layer sizes of Qwen3-8B on inputs larger than
the L2 cache (weights and pages rotate), holding a few GB at most, and ends by itself in seconds;
it reports the mean CUDA-event time of a launch with the bytes or operations per second that this
makes.  The summaries under profiles/ name the command.
"""

from __future__ import annotations

import argparse

import torch

from .kernels.ops import QUERY_TILE
from .kernels import ops


def _time(fn, reps: int) -> float:
    for i in range(3):
        fn(i)
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(reps):
        fn(3 + i)
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps * 1e3


def gemm_case(M: int, N: int, K: int, reps: int, plan: tuple | None = None) -> dict:
    copies = max(2, int(400e6 // (N * K * 2)) + 1)
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: ops.gemm_tc(x, ws[i % copies], out, plan), reps)
    plan = plan or ops.gemm_tc_plan(M, N, K)
    print(f"gemm_tc M={M} N={N} K={K} plan(swap, bn, splits)={plan}: {us:.1f} us, "
          f"{N * K * 2 / us / 1e3:.0f} GB/s of weights, {2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    return {"kernel": "gemm_tc", "M": M, "N": N, "K": K, "us": us, "weights_gbs": N * K * 2 / us / 1e3,
            "tflops": 2 * M * N * K / us / 1e6}


def attention_case(batch: int, q_len: int, context: int, reps: int, legacy: bool = False, page: int = 64) -> dict:
    NH, NKV, D = 32, 8, 128
    pages_per = (context + page - 1) // page
    n_pages = batch * pages_per
    # rotate over so many pools that a launch finds nothing of its pages in L2 (126 MB): 600 MB in all, three at least
    sets = max(3, -(-600_000_000 // (2 * n_pages * NKV * page * D * 2)))
    pools = [(torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16),
              torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16)) for _ in range(sets)]
    table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(batch, pages_per)
    T = batch * q_len
    qkv = torch.randn(T, (NH + 2 * NKV) * D, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(T, NH * D, device="cuda", dtype=torch.bfloat16)
    kv_len = torch.full((batch,), context, dtype=torch.int32, device="cuda")
    cu_q = (torch.arange(batch + 1, dtype=torch.int32, device="cuda") * q_len)
    if q_len == 1:
        rows = torch.arange(batch, dtype=torch.int32, device="cuda")
        splits, in_clusters = ops.decode_plan(batch, NH, NKV, D, page, context)
        fn = lambda i: ops.attention_decode(qkv, out, *pools[i % sets], rows, rows, batch, kv_len, table, NH, NKV, D,
                                            D ** -0.5, 0, splits, context, cluster_merge=in_clusters)
        us = _time(fn, reps)
        gb = batch * context * NKV * D * 2 * 2 / 1e9
        print(f"attention_decode batch={batch} context={context} page={page} splits={splits}{' in clusters' if in_clusters else ''}: {us:.1f} us, {gb / us * 1e6:.0f} GB/s of pages")
        return {"kernel": "attention_decode", "batch": batch, "context": context, "us": us, "pages_gbs": gb / us * 1e6}
    else:
        tiles = [(b, s) for b in range(batch) for s in range(0, q_len, QUERY_TILE)][::-1]
        tile_seq = torch.tensor([t[0] for t in tiles], dtype=torch.int32, device="cuda")
        tile_q0 = torch.tensor([t[1] for t in tiles], dtype=torch.int32, device="cuda")
        kernel = ops.attention_chunk if legacy else ops.attention_tc
        fn = lambda i: kernel(qkv, out, *pools[i % sets], tile_seq, tile_q0, len(tiles), cu_q, kv_len, table, NH, NKV,
                              D, D ** -0.5, 0)
        us = _time(fn, reps)
        flops = batch * 4.0 * NH * D * (q_len * (context - q_len) + q_len * (q_len + 1) / 2)
        print(f"{kernel.__name__} batch={batch} q_len={q_len} context={context} page={page}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s")
        return {"kernel": kernel.__name__, "batch": batch, "q_len": q_len, "context": context, "us": us, "tflops": flops / us / 1e6}


def decode_split_case(reps: int) -> dict:
    """The split-KV kernel with every way of cutting the context that ``ops.decode_plan`` chooses from, for a few
    batches and context lengths (Qwen3-8B head sizes, pages of 64, rotating pools larger than L2): microseconds a
    launch, with the time the plan reckons and the way it takes."""
    NH, NKV, D, page = 32, 8, 128, 64
    out = {}
    for batch, context in ((1, 8192), (2, 8192), (4, 8192), (4, 16384), (8, 2048), (8, 8192), (12, 8192), (32, 8192), (1, 65536)):
        pages_per = context // page
        n_pages = batch * pages_per
        sets = max(3, -(-600_000_000 // (2 * n_pages * NKV * page * D * 2)))       # 600 MB in all: nothing is found in L2
        pools = [(torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16),
                  torch.randn(n_pages, NKV, page, D, device="cuda", dtype=torch.bfloat16)) for _ in range(sets)]
        table = torch.randperm(n_pages, device="cuda").to(torch.int32).view(batch, pages_per)
        qkv = torch.randn(batch, (NH + 2 * NKV) * D, device="cuda", dtype=torch.bfloat16)
        o = torch.empty(batch, NH * D, device="cuda", dtype=torch.bfloat16)
        kv_len = torch.full((batch,), context, dtype=torch.int32, device="cuda")
        rows = torch.arange(batch, dtype=torch.int32, device="cuda")
        chosen = ops.decode_plan(batch, NH, NKV, D, page, context)
        cells = []
        for reckoned, n_splits, cluster, _ in ops.decode_ways(batch, NH, NKV, D, page, context):
            fn = lambda i: ops.attention_decode(qkv, o, *pools[i % sets], rows, rows, batch, kv_len, table, NH, NKV, D,
                                                D ** -0.5, 0, n_splits, context, cluster_merge=cluster)
            us = min(_time(fn, max(reps, sets)), _time(fn, max(reps, sets)))
            name = f"{n_splits}{'c' if cluster else 's' if n_splits > 1 else ''}"
            out[f"b{batch} c{context} {name}"] = us
            cells.append(f"{name}{'*' if (n_splits, cluster) == chosen else ''} {us:.0f}/{reckoned:.0f}")
        print(f"batch {batch:2d} context {context:6d}: " + "  ".join(cells))
        del pools
        torch.cuda.empty_cache()
    print("   (splits, c = merged inside a cluster, s = through scratch memory, * = the plan's choice: measured / reckoned us)")
    return out


def tile_width_case(reps: int) -> dict:
    """The tokens-on-rows product at every tile width, for the shapes of a 2048-token prefill (8B sizes) and of a
    1024-token portion beside 32 decoding requests (14B sizes): what ``ops.GEMM_TILE_OVERHEAD`` was read from."""
    out = {}
    for M, N, K in ((2048, 4096, 4096), (2048, 4096, 12288), (2048, 24576, 4096), (1056, 5120, 5120), (1056, 5120, 17408),
                    (1056, 34816, 5120)):
        for bn in ops.GEMM_TILE_WIDTHS:
            out[f"{M}x{N}x{K} bn={bn}"] = gemm_case(M, N, K, reps, plan=(0, bn, 1, 8))["us"]
        print(f"   chosen for {M}x{N}x{K}: {ops.gemm_tc_plan(M, N, K)[1]} columns")
    return out


def pair_case(reps: int) -> dict:
    """The tokens-on-rows product with a CTA to a tile of 128 x 256 and with a pair of CTAs to a tile of 256 x 256
    (tcgen05 ``cta_group::2``), launch by launch in turn so that both see the same clocks: the shapes of a prompt of
    2048 and of 8192 tokens (8B sizes) and of a 1024-token portion beside 32 decoding requests (14B sizes)."""
    out = {}
    single, pair = (0, 256, 1, 8), (0, 256, 1, 6, ops.GEMM_PAIR)
    for M, N, K, swiglu in ((2048, 6144, 4096, False), (2048, 4096, 4096, False), (2048, 24576, 4096, True), (2048, 4096, 12288, False),
                            (8192, 6144, 4096, False), (8192, 24576, 4096, True), (8192, 4096, 12288, False),
                            (1056, 5120, 5120, False), (1056, 34816, 5120, True), (512, 4096, 12288, False)):
        copies = max(2, int(300e6 // (N * K * 2)) + 1)
        ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
        res = torch.empty(M, N // 2 if swiglu else N, device="cuda", dtype=torch.bfloat16)
        times = {single: [], pair: []}
        n = 0
        for it in range(3 + 2 * reps):
            for plan in (single, pair):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                ops.gemm_tc(x, ws[n % copies], res, plan, swiglu_pairs=swiglu, static_weights=True)
                b.record()
                n += 1
                if it >= 3:
                    times[plan].append((a, b))
        torch.cuda.synchronize()
        med = {plan: sorted(a.elapsed_time(b) for a, b in ev)[len(ev) // 2] * 1e3 for plan, ev in times.items()}
        chosen = ops.gemm_tc_plan(M, N, K)
        print(f"gemm_tc M={M} N={N} K={K}{' SiLU(gate)*up' if swiglu else ''}: a CTA to a tile {med[single]:.1f} us "
              f"({2 * M * N * K / med[single] / 1e6:.0f} TFLOP/s), a pair {med[pair]:.1f} us ({2 * M * N * K / med[pair] / 1e6:.0f} TFLOP/s); "
              f"the plan takes {'the pair' if len(chosen) > 4 and chosen[4] == ops.GEMM_PAIR else f'tiles of {chosen[1]} columns'}")
        out[f"{M}x{N}x{K}"] = {"single_us": med[single], "pair_us": med[pair]}
    return out


def sample_case(rows: int, vocab: int, reps: int) -> dict:
    """Temperature 0.7 and top-p 0.9 over rows of a real vocabulary (a cluster of CTAs shares a row)."""
    logits = [torch.randn(rows, vocab, device="cuda") * 3.0 for _ in range(4)]
    f = lambda v: torch.full((rows,), v, device="cuda", dtype=torch.float32)
    temp, top_p, min_p = f(0.7), f(0.9), f(0.0)
    top_k = torch.zeros(rows, device="cuda", dtype=torch.int32)
    seed = torch.arange(rows, device="cuda", dtype=torch.int64)
    out = torch.empty(rows, device="cuda", dtype=torch.int32)
    counter = torch.zeros(rows, device="cuda", dtype=torch.int64)
    us = _time(lambda i: ops.sample(logits[i % 4], temp, top_k, top_p, min_p, seed, counter, out), reps)
    print(f"sample rows={rows} vocab={vocab} temperature 0.7 top-p 0.9: {us:.1f} us")
    return {"kernel": "sample", "rows": rows, "vocab": vocab, "us": us}


def decode_layer_case(batch: int, context: int, reps: int, fused: bool) -> dict:
    """One layer of the Qwen3-8B sizes in a decode step of ``batch`` requests: the persistent kernel, or the seven
    separate launches, on the same inputs (weights rotate over three layers so that none is found in L2)."""
    from .config import Qwen3Config
    from .engine.batch import StepEntry
    from .engine.runner import ModelRunner
    from .models import build_random
    cfg = Qwen3Config(vocab_size=2048, hidden_size=4096, intermediate_size=12288, num_hidden_layers=3, num_attention_heads=32,
                      num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1e6, max_position_embeddings=16384, tie_word_embeddings=False)
    model = build_random(cfg, 0, torch.bfloat16, "cuda:0")
    for b in model.blocks:
        b.fuse_decode = fused
    page = 16
    runner = ModelRunner(model, page, batch * (context + 256) // page + 8, batch, max_len=context + 256)
    runner.enable_graphs()          # as serving runs decode steps: replayed from a captured graph
    names = [f"r{i}" for i in range(batch)]
    ids = [(7 * i + 3) % 2000 + 5 for i in range(context)]
    for n in names:
        for pos in range(0, context, 2048):
            runner.step([StepEntry(n, ids[pos:pos + 2048], ())])
    entries = [StepEntry(n, [11], (0,)) for n in names]
    us = _time(lambda i: runner.step(entries), reps) / 3.0
    runner.check_status()
    if fused:       # when each CTA finished each phase of the last layer that ran (device-wide nanosecond timer)
        ops.DECODE_LAYER_TRACE = torch.zeros(ops.sm_count(), 8, dtype=torch.int64, device="cuda")
        runner.graphs = None        # a captured graph holds the arguments it was captured with: this one step runs eagerly
        runner.step(entries)
        torch.cuda.synchronize()
        t = ops.DECODE_LAYER_TRACE.cpu().numpy()
        ops.DECODE_LAYER_TRACE = None
        rel = (t - t[:, 0].min()) / 1e3
        names_ph = ["begin", "norm", "q/k/v", "attention", "output", "norm", "gate/up", "down"]
        print("phase ends, us after the first CTA began (earliest..latest CTA): " +
              "  ".join(f"{n} {rel[:, i].min():.1f}..{rel[:, i].max():.1f}" for i, n in enumerate(names_ph)))
    print(f"decode layer ({'one persistent kernel' if fused else 'separate launches'}) batch={batch} context={context}: "
          f"{us:.1f} us a layer (the step's embedding, final norm and head included, divided by 3 layers)")
    return {"kernel": "decode_layer" if fused else "separate", "batch": batch, "context": context, "us_per_layer": us}


CASES = {
    "gemm_decode": lambda r: gemm_case(8, 6144, 4096, r),
    "gemm_decode_mlp": lambda r: gemm_case(8, 24576, 4096, r),
    "gemm_decode_b64": lambda r: gemm_case(64, 24576, 4096, r),
    "gemm_prefill": lambda r: gemm_case(2048, 24576, 4096, r),
    "attention_decode": lambda r: attention_case(8, 1, 2048, r),
    "attention_decode_b64": lambda r: attention_case(64, 1, 2048, r),
    "attention_decode_32k": lambda r: attention_case(8, 1, 32768, r),
    "attention_decode_b1_128k": lambda r: attention_case(1, 1, 131072, r),
    "attention_prefill": lambda r: attention_case(1, 2048, 2048, r),
    "attention_prefill_8k": lambda r: attention_case(1, 2048, 8192, r),
    "attention_prefill_mma_sync": lambda r: attention_case(1, 2048, 2048, r, legacy=True),
    "gemm_prefill_down": lambda r: gemm_case(2048, 4096, 12288, r),
    "attention_decode_splits": decode_split_case,
    "gemm_tile_widths": tile_width_case,
    "gemm_pairs": pair_case,
    "sample": lambda r: sample_case(8, 151936, r),
    "decode_layer_fused": lambda r: decode_layer_case(8, 2048, r, True),
    "decode_layer_separate": lambda r: decode_layer_case(8, 2048, r, False),
}


def bench_kernels(cases=None, reps: int = 6) -> dict:
    """{case: its figures} for the named cases (default: all)."""
    ops.library()
    return {name: CASES[name](reps) for name in (cases or sorted(CASES))}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--reps", type=int, default=6)
    args = ap.parse_args(argv)
    ops.library()
    CASES[args.case](args.reps)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
