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


def gemm_case(M: int, N: int, K: int, reps: int) -> dict:
    copies = max(2, int(400e6 // (N * K * 2)) + 1)
    ws = [torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda i: ops.gemm_tc(x, ws[i % copies], out), reps)
    plan = ops.gemm_tc_plan(M, N, K)
    print(f"gemm_tc M={M} N={N} K={K} plan(swap, bn, splits)={plan}: {us:.1f} us, "
          f"{N * K * 2 / us / 1e3:.0f} GB/s of weights, {2 * M * N * K / us / 1e6:.0f} TFLOP/s")
    return {"kernel": "gemm_tc", "M": M, "N": N, "K": K, "us": us, "weights_gbs": N * K * 2 / us / 1e3,
            "tflops": 2 * M * N * K / us / 1e6}


def attention_case(batch: int, q_len: int, context: int, reps: int, legacy: bool = False, page: int = 64) -> dict:
    NH, NKV, D = 32, 8, 128
    pages_per = (context + page - 1) // page
    n_pages = batch * pages_per
    sets = 3       # rotate over three pools so that a launch finds nothing of its pages in L2
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
        splits = ops.decode_splits(batch, NKV, context)
        fn = lambda i: ops.attention_decode(qkv, out, *pools[i % sets], rows, rows, batch, kv_len, table, NH, NKV, D,
                                            D ** -0.5, 0, splits, context)
        us = _time(fn, reps)
        gb = batch * context * NKV * D * 2 * 2 / 1e9
        print(f"attention_decode batch={batch} context={context} page={page} splits={splits}: {us:.1f} us, {gb / us * 1e6:.0f} GB/s of pages")
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


CASES = {
    "gemm_decode": lambda r: gemm_case(8, 6144, 4096, r),
    "gemm_decode_mlp": lambda r: gemm_case(8, 24576, 4096, r),
    "gemm_decode_b64": lambda r: gemm_case(64, 24576, 4096, r),
    "gemm_prefill": lambda r: gemm_case(2048, 24576, 4096, r),
    "attention_decode": lambda r: attention_case(8, 1, 2048, r),
    "attention_decode_b64": lambda r: attention_case(64, 1, 2048, r),
    "attention_prefill": lambda r: attention_case(1, 2048, 2048, r),
    "attention_prefill_8k": lambda r: attention_case(1, 2048, 8192, r),
    "attention_prefill_mma_sync": lambda r: attention_case(1, 2048, 2048, r, legacy=True),
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
