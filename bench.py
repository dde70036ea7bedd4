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


def _free_device_memory() -> None:
    import gc

    import torch
    gc.collect()
    torch.cuda.empty_cache()


def run_ours(args) -> int:
    import torch

    from acvram_b200 import Engine, SamplingParams
    from acvram_b200 import bench as B
    from acvram_b200.config import Qwen3Config
    from acvram_b200.kernels import ops
    from acvram_b200.models import build_random

    t_begin = time.time()
    pk, pk_src = peaks()
    K, W = args.steps, args.warmup
    page = args.page_size
    refused: dict[str, str] = {}
    points: dict[str, float] = {}

    def build(shape_name: str, layers: int | None, max_batch: int, pool_tokens: int, max_model_len: int, budget: int = 4096):
        shape = SHAPES[shape_name]
        cfg = Qwen3Config(**{**shape, "num_hidden_layers": layers or shape["num_hidden_layers"]})
        t0 = time.time()
        model = build_random(cfg, seed=0, dtype=torch.bfloat16, device="cuda:0")
        torch.cuda.synchronize()
        print(f"[bench] {shape_name}: model built in {time.time() - t0:.1f} s ({model.weight_bytes() / 1e9:.2f} GB)",
              file=sys.stderr, flush=True)
        engine = Engine(model, "bfloat16", max_batch_size=max_batch, max_model_len=max_model_len, page_size=page,
                        num_pages=pool_tokens // page + 2 * max_batch + 8, token_budget=budget,
                        enable_cuda_graphs=not args.no_cuda_graphs,
                        enable_prefix_cache=False)     # every prompt is computed: no number rests on pages taken over
        return cfg, model, engine

    def decode_point(runner, batch: int, context: int, steps: int, warmup: int, sample_clocks: bool = False):
        names = [f"d{batch}-{context}-{i}" for i in range(batch)]
        B.fill_contexts(runner, names, context)
        torch.cuda.synchronize()
        try:
            if sample_clocks:
                with B.ClockSampler() as cs:
                    res = B.time_decode(runner, names, steps, warmup)
                res["clocks"] = cs.summary()
            else:
                res = B.time_decode(runner, names, steps, warmup)
        finally:
            for n in names:
                runner.release(n)
        mid = context + warmup + steps // 2
        res["bytes"] = B.decode_step_bytes(runner.model, batch, mid)
        res["gbs"] = res["bytes"] / (res["ms_per_step"] * 1e-3) / 1e9
        return res

    def point(name: str, fn) -> None:
        """One further point: its number, or why it was refused; never the end of the run."""
        try:
            fn()
        except B.Refused as exc:
            refused[name] = str(exc)
        except Exception as exc:  # noqa: BLE001  (a point beside the headline must not cost the headline)
            refused[name] = f"{type(exc).__name__}: {exc}"[:200]

    # ------------------------------------------------------------------ the headline shape
    shape = SHAPES[args.shape]
    full_layers = shape["num_hidden_layers"]
    layers = args.layers or full_layers
    fill_steps = -(-args.batch * args.context // 4096)        # steps in which the end-to-end run's prompts are computed
    per_request = args.context + 2 * (K + W) + fill_steps + 3 * page
    max_batch = max(args.batch, 64 if not args.skip_points else args.batch)
    long_ctx = 8192
    cfg, model, engine = build(args.shape, layers, max_batch, max_batch * per_request + 2048 + page, 8192)
    runner = engine.runner

    try:
        main = decode_point(runner, args.batch, args.context, K, W, sample_clocks=True)
    except B.Refused as exc:
        print(json.dumps({"metric": f"decode tok/s at batch {args.batch}", "value": None, "refused": str(exc), "n_gpus": 1,
                          "steps": K, "warmup": W}))
        return 3

    # end to end through the public entry point: host ids in, host ids out, every step
    def end_to_end(sp_of) -> tuple[float, int]:
        for i in range(args.batch):
            engine.add_request(B.synthetic_ids(cfg.vocab_size, args.context, 50 + i), sp_of(i))
        while any(r.remaining > 1 or r.computed == 0 for r in engine.scheduler.running) or engine.scheduler.waiting:
            engine.step()
        for _ in range(W):
            engine.step()
        torch.cuda.synchronize()
        replays0 = runner.graphs.replays if runner.graphs is not None else 0
        t0 = time.perf_counter()
        got = 0
        for _ in range(K):
            got += sum(len(o.token_ids) for o in engine.step())
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        h2d = runner.builder.last_h2d_bytes
        replayed = (runner.graphs.replays - replays0) if runner.graphs is not None else K
        while not engine.idle:
            engine.step()
        if got != K * args.batch:
            raise B.Refused(f"{got} tokens came out of {K} steps of {args.batch} requests")
        if engine.stats.failed_steps:
            raise B.Refused(f"a step failed: {engine.last_error}")
        if runner.graphs is not None and runner.graphs.disabled_reason is None and replayed < K:
            raise B.Refused(f"{K - replayed} of {K} timed steps did not replay a captured graph")
        return got / dt, h2d

    # requests whose prompts are done decode while the others' prompts are computed: enough tokens for those steps too
    n_out = K + W + 4 + fill_steps
    graphs_on = bool(engine.enable_cuda_graphs)
    try:
        e2e_rate, h2d = end_to_end(lambda i: SamplingParams(temperature=0.0, max_tokens=n_out, ignore_eos=True))
        e2e = {"value": round(e2e_rate, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch + 4}
    except B.Refused as exc:
        e2e = {"value": None, "unit": "tokens/s", "refused": str(exc)}
    # one prompt of 2048 tokens (a different one each time): 3 untimed, then the median of 5
    pre = B.time_prefill(runner, 2048, reps=5, warmup=3)
    pre_frac = B.prefill_flops(model, 2048) / (pre["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12)

    if not args.skip_points:
        for b in (1, 64):
            def f(b=b):
                r = decode_point(runner, b, args.context, K, W)
                points[f"decode_b{b}"] = round(r["tokens_per_s"], 1)
                points[f"decode_b{b}_hbm_frac"] = round(r["gbs"] / pk["hbm_gbs"], 4)
            point(f"decode_b{b}", f)

    if not args.skip_points:
        def sampled():
            rate, _ = end_to_end(lambda i: SamplingParams(temperature=0.7, top_p=0.9, max_tokens=n_out, ignore_eos=True, seed=i))
            points[f"sampled_b{args.batch}_e2e"] = round(rate, 1)
        point("sampled_e2e", sampled)

        def long_context():
            # contexts of 8192 tokens need room beyond the headline engine's 8192: a runner of its own on the same model
            from acvram_b200.engine.runner import ModelRunner
            nonlocal engine, runner
            del engine, runner
            _free_device_memory()
            tokens = args.batch * (long_ctx + 2 * (K + W) + 3 * page) + long_ctx + page
            long_runner = ModelRunner(model, page, tokens // page + 8, args.batch + 1, max_len=2 * long_ctx)
            if not args.no_cuda_graphs:
                long_runner.enable_graphs()
            r = decode_point(long_runner, args.batch, long_ctx, K, W)
            points[f"decode_b{args.batch}_ctx{long_ctx}"] = round(r["tokens_per_s"], 1)
            points[f"decode_b{args.batch}_ctx{long_ctx}_hbm_frac"] = round(r["gbs"] / pk["hbm_gbs"], 4)
            p8 = B.time_prefill(long_runner, long_ctx, reps=3, warmup=1)
            points[f"prefill_{long_ctx}"] = round(p8["tokens_per_s"], 1)
            points[f"prefill_{long_ctx}_frac"] = round(B.prefill_flops(model, long_ctx) / (p8["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
        point("long_context", long_context)

    line = {
        "metric": f"decode tok/s at batch {args.batch} (Qwen3-{args.shape.upper()} shape, {args.context}-token contexts)",
        "value": round(main["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(main["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic token ids, random weights N(0,0.02)",
        "config": bench_config(args, cfg.to_dict(), layers, full_layers, page, graphs_on),
        "clocks": main.get("clocks"),
        "e2e": e2e,
        "gpu_launches": main["launches"],
        "prefill": {"value": round(pre["tokens_per_s"], 1), "tokens": 2048, "ms": round(pre["ms"], 3),
                    "frac": round(pre_frac, 4), "peak_tflops": pk["bf16_tflops"], "peaks": pk_src,
                    # the same against what cuBLAS holds back to back for seconds under the power cap: a prompt's
                    # step is 26 ms of dense products, run eight times in a row here
                    "frac_of_sustained": round(pre_frac * pk["bf16_tflops"] / pk["bf16_tflops_sustained"], 4)},
        "roofline": {"bound": "hbm", "achieved": round(main["gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(main["gbs"] / pk["hbm_gbs"], 4), "peaks": pk_src},
        "points": points,
    }

    # ------------------------------------------------------------------ the other shapes that the baseline names
    if not args.skip_points and args.shape == "8b" and not args.layers:
        engine = runner = model = None
        _free_device_memory()

        def shape_14b():
            # a step of serving under load: 32 requests decode beside a 1024-token portion of another's prompt
            _, model14, eng14 = build("14b", None, 40, 33 * (2048 + 2 * (K + W) + 64) + 4096, 8192)
            try:
                names = [f"m{i}" for i in range(32)]
                B.fill_contexts(eng14.runner, names, 2048)
                r = B.time_mixed(eng14.runner, names, 1024, 2048, K, W)
                cost = model14.step_cost([1] * 32 + [1024], [2048 + W + K // 2] * 32 + [1536], 33)
                points["mixed_14b_32dec_1024_ms"] = round(r["ms_per_step"], 3)
                points["mixed_14b_32dec_1024_tok_s"] = round(r["tokens_per_s"], 1)
                points["mixed_14b_tflops_frac"] = round(cost["flops"] / (r["ms_per_step"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
            finally:
                del eng14, model14
                _free_device_memory()
        if time.time() - t_begin < args.time_limit:
            point("mixed_14b", shape_14b)
        else:
            refused["mixed_14b"] = "left out: the run's time limit was reached"

        def shape_32b():
            _, model32, eng32 = build("32b", None, 64, 64 * (2048 + 2 * (K + W) + 64) + 4096, 16384)
            try:
                for b in (1, 8, 64):
                    r = decode_point(eng32.runner, b, 2048, K, W)
                    points[f"decode_32b_b{b}"] = round(r["tokens_per_s"], 1)
                    points[f"decode_32b_b{b}_hbm_frac"] = round(r["gbs"] / pk["hbm_gbs"], 4)
                p32 = B.time_prefill(eng32.runner, 2048, reps=3, warmup=1)
                points["prefill_32b_2048"] = round(p32["tokens_per_s"], 1)
                points["prefill_32b_2048_frac"] = round(B.prefill_flops(model32, 2048) / (p32["ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)
            finally:
                del eng32, model32
                _free_device_memory()
        if time.time() - t_begin < args.time_limit:
            point("shape_32b", shape_32b)
        else:
            refused["shape_32b"] = "left out: the run's time limit was reached"

    if refused:
        line["refused"] = refused
    print(json.dumps(line))
    return 0


def bench_config(args, cfg, layers: int, full_layers: int, page: int, graphs: bool) -> dict:
    """The configuration's sizes, flat, the same keys in both arms (the reference arm fills what it knows)."""
    return {"model": f"Qwen3-{args.shape.upper()} shape", "layers": layers, "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "q_heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": args.batch,
            "seq_len": args.context, "max_model_len": 8192, "page_size": page, "kv_dtype": "bf16",
            "prefill_tokens": 2048, "parallelism": "single GPU",
            "l2": "inputs larger than L2 (weights + cache read per step >> 126 MB)", "cuda_graphs": graphs}


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
    ap.add_argument("--time-limit", type=float, default=240.0,
                    help="seconds after which the points at the 14B and 32B layer sizes are left out (and named as left out)")
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
