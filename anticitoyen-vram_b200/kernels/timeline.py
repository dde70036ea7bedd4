"""Device timeline of a step: when every CTA of every kernel began and ended.

A diagnostic build of the kernels (environment variable ``ACVRAM_B200_TIMELINE=1`` before the first
import; it compiles to a library of its own) logs, per CTA, the device-wide nanosecond timer at
its begin and end.  This module reads the logs, groups the records into launches and prints where
the time of a step goes: each launch's span, how long after its predecessor's end it began
(negative when they overlap), and how long its CTAs ran.  Unlike a profiler's launch list it
shows the step as it runs in serving: inside the CUDA graph, with overlapping launches and warm
caches.

    ACVRAM_B200_TIMELINE=1 python -m acvram_b200.kernels.timeline --layers 4 --batch 8 --context 2048
"""

from __future__ import annotations

import argparse
import ctypes
import sys

import numpy as np

from . import ops

MARKS = 12
RECORD = np.dtype([("t0", "<u8"), ("t1", "<u8"), ("kernel", "<i4"), ("block", "<i4"), ("grid", "<i4"), ("smid", "<i4"),
                   ("mark", "<u8", (MARKS,)), ("cycles", "<u8")])
FILES = ("gemm_tc", "elementwise", "sampling", "attention_decode", "attention_tc", "qk_rope_append")
NAMES = {1: "gemm", 2: "norm", 3: "rope_append", 4: "attn_decode", 5: "attn_prompt", 6: "attn_chunk", 7: "embed",
         8: "argmax", 9: "swiglu"}
MARK_NAMES = {1: ("first_full", "last_mma", "acc_done", "part_sent", "cluster_met", "stored", "wait_over", "staged"),
              4: ("loop_done",)}
# the prompt attention's marks are not times but sums: nanoseconds its first softmax warp spent in each phase
# (marks 0..4) and the number of half tiles of 64 keys it went through (mark 7)
ATTN_PHASES = ("wait for S", "row maximum", "rescale O", "exponentials + pack + write P", "hand P over")
CAP = 1 << 16


def enabled() -> bool:
    return hasattr(ops.library(), "acv_tl_read_gemm_tc")


def read(reset: bool = True) -> np.ndarray:
    """All records logged since the last reset, ordered by begin time."""
    lib = ops.library()
    if not enabled():
        raise RuntimeError("the kernels were built without the timeline; set ACVRAM_B200_TIMELINE=1 before importing")
    parts = []
    for f in FILES:
        fn = getattr(lib, f"acv_tl_read_{f}")
        fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
        fn.restype = ctypes.c_int
        buf = np.zeros(CAP, dtype=RECORD)
        n = fn(buf.ctypes.data, CAP, 1 if reset else 0)
        if n < 0:
            raise RuntimeError(f"reading the timeline of {f} failed")
        parts.append(buf[:n])
    rec = np.concatenate(parts)
    return rec[np.argsort(rec["t0"], kind="stable")]


def launches(rec: np.ndarray) -> list[dict]:
    """Group CTA records into launches: same kernel and grid size, blocks not yet seen."""
    out: list[dict] = []
    open_by_key: dict = {}
    for r in rec:
        key = (int(r["kernel"]), int(r["grid"]))
        cur = open_by_key.get(key)
        if cur is None or int(r["block"]) in cur["blocks"] or len(cur["blocks"]) == cur["grid"]:
            cur = {"kernel": key[0], "grid": key[1], "blocks": set(), "t0": [], "t1": [], "marks": []}
            open_by_key[key] = cur
            out.append(cur)
        cur["blocks"].add(int(r["block"]))
        cur["t0"].append(int(r["t0"]))
        cur["t1"].append(int(r["t1"]))
        cur["marks"].append([int(m) for m in r["mark"]])
    for L in out:
        L["begin"], L["end"] = min(L["t0"]), max(L["t1"])
        L["first_end"] = min(L["t1"])
        L["last_begin"] = max(L["t0"])
        L["events"] = {}
        for i, name in enumerate(MARK_NAMES.get(L["kernel"], ())):
            vals = [m[i] for m in L["marks"] if m[i]]
            if vals:
                L["events"][name] = vals
    out.sort(key=lambda L: L["begin"])
    return out


def report(rec: np.ndarray, file=sys.stdout) -> None:
    Ls = launches(rec)
    if not Ls:
        print("no records", file=file)
        return
    origin = Ls[0]["begin"]
    print(f"{'kernel':<12} {'grid':>5} {'begin':>9} {'gap':>7} {'span':>7} {'ramp':>6} {'tail':>6}  events (us after begin: min..max)",
          file=file)
    prev_end = None
    totals: dict = {}
    for L in Ls:
        us = lambda t: (t - origin) / 1e3
        span = (L["end"] - L["begin"]) / 1e3
        gap = (L["begin"] - prev_end) / 1e3 if prev_end is not None else 0.0
        ramp = (L["last_begin"] - L["begin"]) / 1e3          # last CTA's begin after the first's
        tail = (L["end"] - L["first_end"]) / 1e3             # last CTA's end after the first's
        ev = " ".join(f"{k}:{(min(v) - L['begin']) / 1e3:.1f}..{(max(v) - L['begin']) / 1e3:.1f}"
                      for k, v in L["events"].items())
        name = NAMES.get(L["kernel"], str(L["kernel"]))
        print(f"{name:<12} {L['grid']:>5} {us(L['begin']):>9.1f} {gap:>7.1f} {span:>7.1f} {ramp:>6.1f} {tail:>6.1f}  {ev}",
              file=file)
        t = totals.setdefault(name, [0, 0.0, 0.0])
        t[0] += 1
        t[1] += span
        t[2] += max(gap, 0.0)
        prev_end = max(prev_end, L["end"]) if prev_end is not None else L["end"]
    attn = rec[rec["kernel"] == 5]
    if len(attn) and attn["mark"][:, 7].sum() > 0:
        tiles = float(attn["mark"][:, 7].sum())
        print("\nprompt attention, softmax warps of head 0, mean ns per half tile of 64 keys (timer reads included): " +
              ", ".join(f"{name} {attn['mark'][:, i].sum() / tiles:.0f}" for i, name in enumerate(ATTN_PHASES)), file=file)
    whole = (max(L["end"] for L in Ls) - origin) / 1e3
    print(f"\nstep: {whole:.1f} us from the first CTA's begin to the last CTA's end", file=file)
    for name, (n, span, gap) in sorted(totals.items(), key=lambda kv: -kv[1][1]):
        print(f"  {name:<12} {n:>4} launches, spans {span:>8.1f} us, idle gaps before them {gap:>7.1f} us", file=file)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--no-cuda-graphs", action="store_true")
    ap.add_argument("--prefill", type=int, default=0, help="record one prompt step of this many tokens instead of a decode step")
    ap.add_argument("--page", type=int, default=64)
    ap.add_argument("--out", default="")
    ap.add_argument("--dump", default="", help="also save the raw records (numpy .npy)")
    args = ap.parse_args(argv)
    import torch
    from .. import bench as B
    from ..config import Qwen3Config
    from ..engine import Engine
    from ..engine.batch import StepEntry
    from ..models import build_random
    cfg = Qwen3Config(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=args.layers,
                      num_attention_heads=32, num_key_value_heads=8, head_dim=128, max_position_embeddings=40960,
                      rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False)
    model = build_random(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    pages = args.batch * (args.context // args.page + 8) + 8
    if args.prefill:
        pages = max(pages, 3 * (args.prefill // args.page + 2))
    engine = Engine(model, "bfloat16", max_batch_size=args.batch, max_model_len=8192, page_size=args.page, num_pages=pages,
                    token_budget=4096, enable_cuda_graphs=not args.no_cuda_graphs)
    runner = engine.runner
    if args.prefill:
        for k in range(3):
            if k == 2:
                torch.cuda.synchronize()
                read(reset=True)
            runner.step([StepEntry(f"p{k}", B.synthetic_ids(cfg.vocab_size, args.prefill, 7 + k), (args.prefill - 1,))])
            runner.release(f"p{k}")
        torch.cuda.synchronize()
        rec = read(reset=True)
    else:
        names = [f"t{i}" for i in range(args.batch)]
        B.fill_contexts(runner, names, args.context)
        tokens = torch.full((args.batch,), 11, dtype=torch.int32, device="cuda:0")
        entries = [StepEntry(n, [0], (0,)) for n in names]
        for _ in range(6):
            ops.argmax(runner.step(entries, device_tokens=tokens), tokens)
        torch.cuda.synchronize()
        read(reset=True)
        for _ in range(2):          # the second step of the two follows a step, as in serving
            ops.argmax(runner.step(entries, device_tokens=tokens), tokens)
        torch.cuda.synchronize()
        rec = read(reset=True)
        # keep the second step: from its embedding launch on
        emb = rec[rec["kernel"] == 7]
        if len(emb) >= 2:
            starts = sorted(set(int(t) for t in emb["t0"]))
            second = [t for t in starts if t - starts[0] > 100_000]
            if second:
                rec = rec[rec["t0"] >= second[0]]
    if args.dump:
        np.save(args.dump, rec)
    out = open(args.out, "w") if args.out else sys.stdout
    report(rec, file=out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
