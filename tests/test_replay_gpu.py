"""Trace replay through bin/trace_run, compared with the plain implementation.

The same requests are replayed whole; with the last 32 tokens one by one; in
portions of changing size down to two tokens; and mixed, up to four live requests,
portions of some beside single tokens of others, in a pool so small that pages are
used again.  In float32 every logit must agree with the plain implementation to
rounding; in bfloat16 the distance is judged against the distance that the plain
implementation itself shows between its bfloat16 and float32 runs.
"""

from __future__ import annotations

import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3
from conftest import ROOT, random_ids

pytestmark = pytest.mark.gpu

TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


# --------------------------------------------------------------------------- building traces
class Trace:
    """Steps for trace_run plus the book of which output row is which (request, position)."""

    def __init__(self):
        self.steps = []       # dicts as trace_run reads them
        self.book = []        # per step: list of (request, position) in output order
        self.fed = {}         # request -> tokens fed so far
        self.live_peak = 0

    def step(self, parts: dict[str, list[int]], end=()):
        """parts: request -> its next tokens; logits are wanted at every place."""
        entries, rows = [], []
        for rid, toks in parts.items():
            start = self.fed.get(rid, 0)
            entries.append({"id": rid, "tokens": list(toks), "want": list(range(len(toks)))})
            rows += [(rid, start + i) for i in range(len(toks))]
            self.fed[rid] = start + len(toks)
        live = sum((n + 63) // 64 * 64 for n in self.fed.values())
        self.live_peak = max(self.live_peak, live)
        self.steps.append({"step": len(self.steps), "entries": entries, "end": list(end)})
        self.book.append(rows)
        for rid in end:
            del self.fed[rid]


def play_whole(tr: Trace, reqs: dict[str, list[int]], tag: str):
    for rid, ids in reqs.items():
        tr.step({f"{tag}{rid}": ids}, end=[f"{tag}{rid}"])


def play_tail(tr: Trace, reqs, tag: str, tail: int = 32):
    for rid, ids in reqs.items():
        name = f"{tag}{rid}"
        head = max(1, len(ids) - tail) if len(ids) > 1 else 1
        tr.step({name: ids[:head]}, end=[name] if head == len(ids) else [])
        for i in range(head, len(ids)):
            tr.step({name: ids[i:i + 1]}, end=[name] if i == len(ids) - 1 else [])


def play_portions(tr: Trace, reqs, tag: str, seed: int):
    rng = random.Random(seed)
    for rid, ids in reqs.items():
        name = f"{tag}{rid}"
        pos = 0
        while pos < len(ids):
            n = min(len(ids) - pos, rng.choice([2, 2, 3, 5, 7, 16, 17, 31, 40]))
            if len(ids) - pos - n == 1:   # never leave a lone last token: portions go down to two
                n += 1
            tr.step({name: ids[pos:pos + n]}, end=[name] if pos + n == len(ids) else [])
            pos += n


def play_mixed(tr: Trace, reqs, tag: str, seed: int, max_live: int = 4, tail: int = 32):
    """Up to max_live requests at once: prompt portions beside single tokens, some requests left
    out of a step, finished ones ended at once so that later ones take their pages."""
    rng = random.Random(seed)
    waiting = [(f"{tag}{rid}", ids) for rid, ids in reqs.items()]
    live: dict[str, tuple[list[int], int]] = {}
    while waiting or live:
        while waiting and len(live) < max_live:
            name, ids = waiting.pop(0)
            live[name] = (ids, 0)
        parts, end = {}, []
        names = list(live)
        rng.shuffle(names)
        for name in names:
            ids, pos = live[name]
            if parts and rng.random() < 0.25:
                continue                     # left out of this step, goes on later
            head = max(1, len(ids) - tail)
            if pos < head:
                n = min(head - pos, rng.choice([2, 3, 5, 8, 13, 24]))
                if head - pos - n == 1:
                    n += 1
            else:
                n = 1
            parts[name] = ids[pos:pos + n]
            live[name] = (ids, pos + n)
            if pos + n == len(ids):
                end.append(name)
        tr.step(parts, end=end)
        for name in end:
            del live[name]


# --------------------------------------------------------------------------- running
def run_trace(folder: str, dtype: str, tr: Trace, out_dir: str, max_tokens: int, page_size: int | None = None) -> dict:
    env = dict(os.environ)
    extra = ["--page-size", str(page_size)] if page_size else []
    proc = subprocess.Popen([sys.executable, TRACE_RUN, "--model", folder, "--dtype", dtype, "--out", out_dir,
                             "--max-tokens", str(max_tokens), *extra], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                            text=True, env=env)
    try:
        for s in tr.steps:
            proc.stdin.write(json.dumps(s) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {s['step']}", f"trace_run answered {line!r} at step {s['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    got: dict[tuple[str, int], np.ndarray] = {}
    for s, rows in zip(tr.steps, tr.book):
        data = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4")
        data = data.reshape(len(rows), -1)
        for row, key in zip(data, rows):
            got[key] = row
    return got


def requests_for(name: str, vocab: int) -> dict[str, list[int]]:
    lengths = {"A": [5, 17, 33, 70, 130], "B": [1, 9, 40, 130, 75], "C": [3, 64, 97, 250], "D": [2, 65, 129, 200, 31], "E": [4, 37, 90],
               "F": [3, 66, 131, 300, 129], "R": [3, 200, 513, 140, 66]}[name]
    return {str(i): random_ids(vocab, n, seed=100 + i) for i, n in enumerate(lengths)}


def build_full_trace(name: str, vocab: int) -> tuple[Trace, dict[str, list[int]], dict[str, str]]:
    reqs = requests_for(name, vocab)
    tr = Trace()
    play_whole(tr, reqs, "w")
    play_tail(tr, reqs, "t")
    play_portions(tr, reqs, "p", seed=7)
    play_mixed(tr, reqs, "m", seed=11)
    play_mixed(tr, reqs, "n", seed=12, max_live=3)
    return tr, reqs, {"w": "whole", "t": "tail one by one", "p": "portions", "m": "mixed", "n": "mixed, 3 live"}


@pytest.fixture(scope="module")
def plain_logits(plain_models):
    cache = {}

    def get(name: str, dtype=torch.float32):
        key = (name, dtype)
        if key not in cache:
            cfg, t = plain_models[name]
            reqs = requests_for(name, cfg["vocab_size"])
            cache[key] = {rid: plain_qwen3.forward_logits(cfg, t, ids, dtype).numpy() for rid, ids in reqs.items()}
        return cache[key]

    return get


def worst(got, ref, modes):
    """max |got - ref| per replay mode, and where the first bad token would be."""
    out = {}
    for (rid, pos), row in got.items():
        mode, req = rid[0], rid[1:]
        d = float(np.abs(row - ref[req][pos]).max())
        if d > out.get(mode, (0.0, None))[0]:
            out[mode] = (d, (req, pos))
    return {modes[m]: v for m, v in out.items()}


@pytest.mark.parametrize("name", ["A", "B", "C", "E", "F"])
def test_replay_float32(name, tiny_folders, plain_logits, tmp_path):
    cfg = json.load(open(os.path.join(tiny_folders[name], "config.json")))
    tr, reqs, modes = build_full_trace(name, cfg["vocab_size"])
    got = run_trace(tiny_folders[name], "float32", tr, str(tmp_path), tr.live_peak)
    ref = plain_logits(name)
    assert len(got) == 5 * sum(len(v) for v in reqs.values())
    report = worst(got, ref, modes)
    scale = max(float(np.abs(v).max()) for v in ref.values())
    for mode, (d, where) in report.items():
        assert d <= 2e-5 * max(1.0, scale), f"{mode}: max |logit - plain| = {d:.3e} at request/position {where}"


@pytest.mark.parametrize("name,page", [("A", None), ("B", None), ("C", None), ("D", None), ("E", None), ("F", None), ("F", 64),
                                       ("D", 32)])
def test_replay_bfloat16(name, page, tiny_folders, plain_logits, tmp_path):
    """page None: trace_run's own page of 16; F and D also with the serving default of 64 and with 32."""
    cfg = json.load(open(os.path.join(tiny_folders[name], "config.json")))
    tr, reqs, modes = build_full_trace(name, cfg["vocab_size"])
    got = run_trace(tiny_folders[name], "bfloat16", tr, str(tmp_path), tr.live_peak, page)
    ref = plain_logits(name)
    ref_bf16 = plain_logits(name, torch.bfloat16)
    # the yardstick: how far the plain implementation's own bfloat16 run is from its float32 run
    yard = max(float(np.abs(ref_bf16[r] - ref[r]).max()) for r in ref)
    report = worst(got, ref, modes)
    for mode, (d, where) in report.items():
        assert d <= 2.5 * yard, (f"{mode}: max |logit - plain| = {d:.3e} at request/position {where}; "
                                 f"plain bf16 vs fp32 is {yard:.3e}")
    # and the modes agree with one another as closely as they agree with the plain run
    whole = {k[0][1:] + f":{k[1]}": v for k, v in got.items() if k[0][0] == "w"}
    for (rid, pos), row in got.items():
        if rid[0] != "w":
            d = float(np.abs(row - whole[rid[1:] + f":{pos}"]).max())
            assert d <= 2.5 * yard, f"{modes[rid[0]]} differs from whole by {d:.3e} at {rid[1:]}/{pos}"


@pytest.fixture(scope="module")
def real_size_model(tmp_path_factory):
    """Two layers with the layer sizes of Qwen3-8B: (folder, config dict, float32 tensors of the plain implementation)."""
    from acvram_b200.weights import write_random_model
    from conftest import TINY_SEEDS, tiny_config
    folder = str(tmp_path_factory.mktemp("real_sizes"))
    write_random_model(tiny_config("R"), folder, TINY_SEEDS["R"])
    return (folder, *plain_qwen3.read_folder(folder))


@pytest.mark.parametrize("dtype,page", [("float32", None), ("bfloat16", None), ("bfloat16", 64)])
def test_replay_at_real_layer_sizes(dtype, page, real_size_model, tmp_path):
    """The four ways of cutting at the layer sizes that serving runs (hidden 4096, 32 query heads on 8 of 128,
    intermediate 12288): the products' tile and split choices, the attention over several tiles of keys."""
    folder, cfg, t = real_size_model
    tr, reqs, modes = build_full_trace("R", cfg["vocab_size"])
    got = run_trace(folder, dtype, tr, str(tmp_path), tr.live_peak, page)
    ref = {rid: plain_qwen3.forward_logits(cfg, t, ids).numpy() for rid, ids in reqs.items()}
    assert len(got) == 5 * sum(len(v) for v in reqs.values())
    report = worst(got, ref, modes)
    if dtype == "float32":
        scale = max(float(np.abs(v).max()) for v in ref.values())
        bound = 2e-5 * max(1.0, scale)
    else:
        ref16 = {rid: plain_qwen3.forward_logits(cfg, t, ids, torch.bfloat16).numpy() for rid, ids in reqs.items()}
        bound = 2.5 * max(float(np.abs(ref16[r] - ref[r]).max()) for r in ref)
    for mode, (d, where) in report.items():
        assert d <= bound, f"{mode}: max |logit - plain| = {d:.3e} at request/position {where} (bound {bound:.3e})"


def test_replay_pages_are_reused(tiny_folders):
    """The mixed trace needs more pages over its life than the pool holds."""
    cfg = json.load(open(os.path.join(tiny_folders["A"], "config.json")))
    tr, reqs, _ = build_full_trace("A", cfg["vocab_size"])
    total = sum((len(v) + 15) // 16 for v in reqs.values())
    assert total * 5 > tr.live_peak // 16
