"""The ``acvram`` command.

Subcommands in the reference's manner (acvram/cli.py:1194-1495 has ``serve``,
``bench``, ``convert`` ... and no ``generate``).  Options that the reference has
keep its names and meanings: ``--max-model-len`` (8192), ``--max-batch`` (16),
``--device``, ``--no-cuda-graphs``, ``--json``, ``bench --what decode``.

    acvram generate MODEL --prompt-ids 1,2,3 --max-tokens 16 --temperature 0
    acvram bench MODEL --what decode --json
    acvram random-model CONFIG.json OUT --seed 0
    acvram replay --model DIR --dtype float32 --out DIR --max-tokens N < steps.jsonl
"""

from __future__ import annotations

import argparse
import json
import sys

from . import __version__


def _engine_args(p: argparse.ArgumentParser, model_optional: bool = False) -> None:
    p.add_argument("model", nargs="?" if model_optional else None,
                   help="model folder (config.json and safetensors), or a config.json with --random-weights")
    p.add_argument("--random-weights", action="store_true", help="ignore the folder's weights; draw them from --seed")
    p.add_argument("--seed", type=int, default=0, help="seed of random weights and of sampling")
    p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    p.add_argument("--max-model-len", type=int, default=8192)
    p.add_argument("--max-batch", type=int, default=16)
    p.add_argument("--page-size", type=int, default=64)
    p.add_argument("--num-pages", type=int, default=None, help="pages of the cache pool (default: from free memory)")
    p.add_argument("--token-budget", type=int, default=2048, help="most tokens that one step runs")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--no-cuda-graphs", action="store_true")
    p.add_argument("--no-prefix-cache", action="store_true",
                   help="compute every prompt from its first token (default: full pages of earlier requests are taken over)")


def _make_engine(args):
    from .engine import Engine
    return Engine(args.model, args.dtype, max_batch_size=args.max_batch, max_model_len=args.max_model_len,
                  page_size=args.page_size, num_pages=args.num_pages, token_budget=args.token_budget,
                  random_weights=args.random_weights, seed=args.seed, device=args.device,
                  enable_cuda_graphs=not args.no_cuda_graphs, enable_prefix_cache=not args.no_prefix_cache)


def cmd_generate(args) -> int:
    from .sampling import SamplingParams
    engine = _make_engine(args)
    vocab = engine.model.plan.vocab_size
    prompts = []
    if args.prompt_ids:
        for spec in args.prompt_ids:
            prompts.append([int(t) for t in spec.replace(",", " ").split()])
    else:
        # the reference's synthetic prompt (acvram/bench.py:375-377)
        for k in range(args.num_prompts):
            prompts.append([(k * 104729 + i * 7919) % max(1, vocab - 100) + 10 for i in range(args.prompt_len)])
    params = SamplingParams(temperature=args.temperature, top_p=args.top_p, top_k=args.top_k, min_p=args.min_p,
                            repetition_penalty=args.repetition_penalty, presence_penalty=args.presence_penalty,
                            frequency_penalty=args.frequency_penalty, max_tokens=args.max_tokens,
                            ignore_eos=args.ignore_eos, seed=args.sampling_seed)
    outs = engine.generate_batch(prompts, params)
    if args.json:
        print(json.dumps({"prompts": prompts, "outputs": outs, "stats": engine.stats.to_dict()}))
    else:
        for p, o in zip(prompts, outs):
            print(" ".join(map(str, o)))
    return 0


def cmd_bench(args) -> int:
    from .bench import bench_decode
    if args.what not in ("all", "decode", "kernels"):
        print(f"bench --what {args.what}: 'decode' and 'kernels' are built", file=sys.stderr)
        return 2
    if args.what == "kernels":
        import contextlib
        from .profile_cases import CASES, bench_kernels
        cases = args.case.split(",") if args.case else None
        unknown = [c for c in cases or () if c not in CASES]
        if unknown:
            print(f"bench --what kernels: no case named {', '.join(unknown)}; there are {', '.join(sorted(CASES))}", file=sys.stderr)
            return 2
        with contextlib.redirect_stdout(sys.stderr if args.json else sys.stdout):
            res = bench_kernels(cases)
        if args.json:
            print(json.dumps(res))
        return 0
    if not args.model:
        print("bench --what decode needs a model folder (or a config.json with --random-weights)", file=sys.stderr)
        return 2
    res = bench_decode(args.model, random_weights=args.random_weights, seed=args.seed, dtype=args.dtype,
                       batches=[int(b) for b in args.batch.split(",")], context=args.context,
                       n_tokens=args.tokens, device=args.device, cuda_graphs=not args.no_cuda_graphs,
                       prefill=args.prefill)
    if args.json:
        print(json.dumps(res))
    else:
        for k, v in res.items():
            print(f"{k}: {v}")
    return 0


def cmd_random_model(args) -> int:
    from .config import load_config
    from .weights import write_random_model
    import torch
    out = write_random_model(load_config(args.config), args.out, args.seed,
                             {"bfloat16": torch.bfloat16, "float32": torch.float32}[args.dtype])
    print(out)
    return 0


def cmd_replay(args) -> int:
    from .engine.replay import replay
    if args.page_size < 1 or 64 % args.page_size:
        raise SystemExit("--page-size must divide 64")
    return replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, sys.stdout, args.device,
                  args.page_size, args.max_requests)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="acvram", description="acvram_b200 - Qwen3 dense inference on one B200")
    p.add_argument("--version", action="version", version=f"acvram_b200 {__version__}")
    sub = p.add_subparsers(dest="command", required=True)

    g = sub.add_parser("generate", help="generate token ids from token ids")
    _engine_args(g)
    g.add_argument("--prompt-ids", action="append", help="comma separated token ids; may be given several times")
    g.add_argument("--prompt-len", type=int, default=128, help="length of synthetic prompts when no ids are given")
    g.add_argument("--num-prompts", type=int, default=1)
    g.add_argument("--max-tokens", type=int, default=512)
    g.add_argument("--temperature", type=float, default=1.0, help="<= 0: greedy")
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--min-p", type=float, default=0.0)
    g.add_argument("--repetition-penalty", type=float, default=1.0)
    g.add_argument("--presence-penalty", type=float, default=0.0)
    g.add_argument("--frequency-penalty", type=float, default=0.0)
    g.add_argument("--sampling-seed", type=int, default=None, help="seed of the requests' generators")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--json", action="store_true")
    g.set_defaults(func=cmd_generate)

    b = sub.add_parser("bench", help="measure decode throughput, or the hot kernels one by one")
    _engine_args(b, model_optional=True)
    b.add_argument("--what", default="decode", help="all | decode | kernels (the reference's names, acvram/cli.py:1476)")
    b.add_argument("--case", default="", help="with --what kernels: the cases to run, comma separated (default: all)")
    b.add_argument("--batch", default="1", help="batch sizes, comma separated")
    b.add_argument("--context", type=int, default=128, help="tokens of context before decoding (reference: 128)")
    b.add_argument("--tokens", type=int, default=256, help="tokens decoded per request (reference: 256)")
    b.add_argument("--prefill", type=int, default=0, help="also time one prompt of this many tokens, computed in one step")
    b.add_argument("--json", action="store_true")
    b.set_defaults(func=cmd_bench)

    r = sub.add_parser("random-model", help="write config.json and model.safetensors with random weights")
    r.add_argument("config", help="a config.json (file or folder)")
    r.add_argument("out")
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    r.set_defaults(func=cmd_random_model)

    t = sub.add_parser("replay", help="feed given token ids step by step and write logits (bin/trace_run)")
    t.add_argument("--model", required=True)
    t.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    t.add_argument("--out", required=True)
    t.add_argument("--max-tokens", type=int, required=True)
    t.add_argument("--device", default="cuda:0")
    t.add_argument("--page-size", type=int, default=16, help="tokens per cache page (a divisor of 64)")
    t.add_argument("--max-requests", type=int, default=16, help="most requests live at a time")
    t.set_defaults(func=cmd_replay)
    return p


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return args.func(args)


if __name__ == "__main__":
    sys.exit(main())
