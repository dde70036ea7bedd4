#!/usr/bin/env python3
"""Headline measurement: decode tokens/s of a Qwen3-8B-shaped model on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

The model has the layer sizes of Qwen3-8B (36 layers, hidden 4096, 32 query and
8 key/value heads of 128, intermediate 12288, vocabulary 151936, rope theta 1e6,
eps 1e-6, untied head) with random weights N(0, 0.02) in bfloat16; the default
run decodes a batch of 8 requests that each hold a 2048-token synthetic context
in a paged bfloat16 cache (pages of 16 tokens, as the baseline's configuration has them).  A step is one decode step of the whole
batch.  One JSON line is printed: ``value`` is decoded tokens per second timed on
the device over exactly K steps after W warm-up steps; ``e2e`` is the same through
``Engine.step()`` with host token ids in and out; ``prefill`` is one 2048-token
prompt; ``roofline`` is the decode step's necessary bytes over its time; ``points``
holds batch 1 and 64.  This program measures one GPU: for --gpus N > 1 it says so
and exits with 2.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

QWEN3_8B = dict(vocab_size=151936, hidden_size=4096, intermediate_size=12288, num_hidden_layers=36,
                num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0,
                max_position_embeddings=40960, tie_word_embeddings=False)
# the larger shapes that the baseline's configurations name, for `--shape`; the default run is the 8B shape
SHAPES = {
    "8b": QWEN3_8B,
    "14b": {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 17408, "num_hidden_layers": 40, "num_attention_heads": 40},
    "32b": {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 25600, "num_hidden_layers": 64, "num_attention_heads": 64},
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    """The roofline's denominators: MEASURED_PEAKS.json beside this file where it exists (its keys are looked
    for at any depth), else the fallback figures."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    found: dict = {}

    def walk(node) -> None:
        if isinstance(node, dict):
            for k, v in node.items():
                if k in FALLBACK_PEAKS and isinstance(v, (int, float)) and not isinstance(v, bool) and v > 0:
                    found.setdefault(k, float(v))
                else:
                    walk(v)
        elif isinstance(node, list):
            for v in node:
                walk(v)

    if os.path.isfile(path):
        try:
            with open(path) as fh:
                walk(json.load(fh))
        except (OSError, ValueError):
            found = {}
    if "hbm_gbs" in found and "bf16_tflops" in found:
        return {**FALLBACK_PEAKS, **found}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def run_reference(args) -> int:
    from baseline.reference_arm import run
    return run(args)


def run_ours(args) -> int:
    import dataclasses

    import torch

    from acvram_b200 import Engine, SamplingParams
    from acvram_b200 import bench as B
    from acvram_b200.config import Qwen3Config
    from acvram_b200.models import build_random

    shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    layers = args.layers or full_layers
    cfg = Qwen3Config(**{**shape, "num_hidden_layers": layers})
    t0 = time.time()
    model = build_random(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.time() - t0:.1f} s ({model.weight_bytes() / 1e9:.2f} GB)", file=sys.stderr)

    K, W = args.steps, args.warmup
    page = args.page_size
    budget = 4096
    fill_steps = -(-args.batch * args.context // budget)        # steps in which the end-to-end run's prompts are computed
    per_request = args.context + 2 * (K + W) + fill_steps + 3 * page
    max_batch = max(args.batch, 64 if not args.skip_points else args.batch)
    num_pages = max_batch * ((per_request + page - 1) // page) + 8 + (2048 + page) // page
    engine = Engine(model, "bfloat16", max_batch_size=max_batch, max_model_len=8192, page_size=page,
                    num_pages=num_pages, token_budget=budget, enable_cuda_graphs=not args.no_cuda_graphs,
                    enable_prefix_cache=False)     # every prompt is computed: no number rests on pages taken over
    runner = engine.runner
    pk, pk_src = peaks()

    def decode_point(batch: int, steps: int, warmup: int, sample_clocks: bool = False):
        names = [f"d{batch}-{i}" for i in range(batch)]
        B.fill_contexts(runner, names, args.context)
        torch.cuda.synchronize()
        if sample_clocks:
            with B.ClockSampler() as cs:
                res = B.time_decode(runner, names, steps, warmup)
            res["clocks"] = cs.summary()
        else:
            res = B.time_decode(runner, names, steps, warmup)
        for n in names:
            runner.release(n)
        return res

    main = decode_point(args.batch, K, W, sample_clocks=True)
    mid_ctx = args.context + W + K // 2
    step_bytes = B.decode_step_bytes(cfg, layers, args.batch, mid_ctx)
    achieved = step_bytes / (main["ms_per_step"] * 1e-3) / 1e9

    # one prompt of 2048 tokens (a different one each time): 3 untimed, then the median of 5
    pre = B.time_prefill(runner, 2048, reps=5, warmup=3)
    flops = B.prefill_flops(cfg, layers, 2048)
    pre_frac = flops / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = round(decode_point(b, K, W)["tokens_per_s"], 1)

    # end to end through the public entry point: host ids in, host ids out, every step
    # requests whose prompts are done decode while the others' prompts are computed: enough tokens for those steps too
    sp = SamplingParams(temperature=0.0, max_tokens=K + W + 4 + fill_steps, ignore_eos=True)
    for i in range(args.batch):
        engine.add_request(B.synthetic_ids(cfg.vocab_size, args.context, 50 + i), sp)
    while any(r.remaining > 1 or r.computed == 0 for r in engine.scheduler.running) or engine.scheduler.waiting:
        engine.step()
    for _ in range(W):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    got = 0
    for _ in range(K):
        got += sum(len(o.token_ids) for o in engine.step())
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    h2d = runner.builder.last_h2d_bytes
    while not engine.idle:
        engine.step()

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.shape.upper()} shape, {args.context}-token contexts)",
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights N(0,0.02)",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": layers, "layers_full": full_layers, "hidden": cfg.hidden_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size, "global_batch": args.batch,
                   "seq_len": args.context, "max_model_len": 8192, "page_size": page, "kv_dtype": "bf16",
                   "prefill_tokens": 2048, "parallelism": "single GPU",
                   "l2": "inputs larger than L2 (weights + cache read per step >> 126 MB)",
                   "cuda_graphs": bool(engine.enable_cuda_graphs)},
        "clocks": main.get("clocks"),
        "e2e": {"value": round(got / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": main["launches"],
        "prefill": {"value": round(pre["tokens_per_s"], 1), "tokens": 2048, "ms": round(pre["ms"], 3),
                    "frac": round(pre_frac, 4), "peak_tflops": pk["bf16_tflops"], "peaks": pk_src},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk_src},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration's (named in config)")
    ap.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="layer sizes (default: Qwen3-8B's)")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--page-size", type=int, default=16, help="tokens in a page of the cache (the engine's own default is 64)")
    ap.add_argument("--skip-points", action="store_true", help="skip the batch 1 and 64 points")
    ap.add_argument("--no-cuda-graphs", action="store_true")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not built (the engine runs on a single device)")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
