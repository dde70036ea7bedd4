"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: it builds
the model as generation does (``build_from_folder``), and every step is one call
of ``ModelRunner.step``.  The reference has no such program; the closest are its
teacher-forced ``logprobs_invite`` (acvram/engine/runner.py:2573-2615) and tests
that drive ``Engine.step()`` by hand (tests/test_prefill_decoupe.py).

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` gets the logits at
the wanted places as little-endian float32 [wanted, vocab].  After every step the
line ``done <step>`` is printed and flushed.
"""

from __future__ import annotations

import json
import os
import sys
from typing import IO

import torch

from .batch import StepEntry
from .runner import ModelRunner

PAGE_SIZE = 16          # the reference's page (acvram/memory/kvcache.py:37)
MAX_LIVE_REQUESTS = 16  # traces hold up to four


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines: IO[str], echo: IO[str],
           device: str = "cuda:0", page_size: int = PAGE_SIZE, max_requests: int = MAX_LIVE_REQUESTS) -> int:
    from ..models import build_from_folder

    run_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    if not torch.cuda.is_available():
        raise RuntimeError("trace_run needs a CUDA device: the engine has no CPU path")
    os.makedirs(out_dir, exist_ok=True)
    _, model = build_from_folder(model_dir, run_dtype, device)
    # every live request's count is rounded up to a multiple of 64 by the caller, and 64 is a
    # multiple of the page, so max_tokens / page_size pages always hold the live requests
    num_pages = (max_tokens + page_size - 1) // page_size
    runner = ModelRunner(model, page_size, num_pages, max_requests)
    if run_dtype == torch.bfloat16:
        runner.enable_graphs()      # as serving does: steps of single tokens replay a captured graph
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", ())]
        logits = runner.step(entries)
        host = logits.to("cpu") if logits.shape[0] else None
        runner.check_status()       # waits for the device; a step whose kernels gave up a wait writes nothing
        if host is not None:
            host.numpy().astype("<f4").tofile(os.path.join(out_dir, f"{step}.f32"))
        for request in rec.get("end", ()):
            if request in runner.manager.lengths:
                runner.release(request)
        print(f"done {step}", file=echo, flush=True)
    return 0


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for the <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--page-size", type=int, default=PAGE_SIZE,
                    help="tokens per cache page (a divisor of 64, so that the rounding of --max-tokens holds)")
    ap.add_argument("--max-requests", type=int, default=MAX_LIVE_REQUESTS, help="most requests live at a time")
    args = ap.parse_args(argv)
    if args.page_size < 1 or 64 % args.page_size:
        ap.error("--page-size must divide 64")
    return replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, sys.stdout, args.device, args.page_size,
                  args.max_requests)
