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
def run_trace(folder: str, dtype: str, tr: Trace, out_dir: str, max_tokens: int, page_size: int | None = None,
              max_requests: int | None = None) -> dict:
    env = dict(os.environ)
    extra = ["--page-size", str(page_size)] if page_size else []
    if max_requests:
        extra += ["--max-requests", str(max_requests)]
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


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E", "F"])
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


# --------------------------------------------------------------------------- the steps that serving runs
def play_serving_steps(tr: Trace, decoders: dict[str, list[int]], bigs: list[tuple[str, list[int], list[int]]]):
    """What a scheduler with a budget of a thousand tokens or two makes: requests that decode, one token each, beside
    a long portion of another request's prompt, in one step.  The decoders' prompts run first, all in one step
    (several portions of a hundred tokens or more side by side); then every portion of every big request runs beside
    one token of each decoder; a big request that ends gives its pages to the next."""
    n_steps = sum(len(portions) for _, _, portions in bigs)
    tr.step({name: ids[:len(ids) - n_steps] for name, ids in decoders.items()})
    at = {name: len(ids) - n_steps for name, ids in decoders.items()}
    k = 0
    for name, ids, portions in bigs:
        assert sum(portions) == len(ids)
        pos = 0
        for n in portions:
            k += 1
            parts = {d: decoders[d][at[d]:at[d] + 1] for d in decoders}
            parts[name] = ids[pos:pos + n]
            pos += n
            end = [name] if pos == len(ids) else []
            if k == n_steps:
                end += list(decoders)
            tr.step(parts, end=end)
            for d in decoders:
                at[d] += 1


SERVING = {   # decoders' lengths; big requests as lists of portions
    "F": ([150, 301, 97], [[600, 129, 171], [257, 443]]),
    "R": ([150, 301, 97], [[1024, 129, 147], [257, 443]]),
}


def bound_for(dtype: str, ref: dict, ref16: dict | None) -> float:
    if dtype == "float32":
        return 2e-5 * max(1.0, max(float(np.abs(v).max()) for v in ref.values()))
    return 2.5 * max(float(np.abs(ref16[r] - ref[r]).max()) for r in ref)


_PLAIN: dict = {}     # the plain implementation's logits, kept between the parametrisations of a test


def plain_cached(cfg, t, ids, dtype=torch.float32):
    key = (json.dumps(cfg, sort_keys=True), tuple(ids), dtype)
    if key not in _PLAIN:
        _PLAIN[key] = plain_qwen3.forward_logits(cfg, t, ids, dtype).numpy()
    return _PLAIN[key]


def check_against_plain(got: dict, reqs: dict[str, list[int]], cfg, t, dtype: str, what: str):
    ref = {rid: plain_cached(cfg, t, ids) for rid, ids in reqs.items()}
    ref16 = None
    if dtype == "bfloat16":
        ref16 = {rid: plain_cached(cfg, t, ids, torch.bfloat16) for rid, ids in reqs.items()}
    bound = bound_for(dtype, ref, ref16)
    assert len(got) == sum(len(v) for v in reqs.values())
    worst_d, where = 0.0, None
    for (rid, pos), row in got.items():
        d = float(np.abs(row - ref[rid][pos]).max())
        if d > worst_d:
            worst_d, where = d, (rid, pos)
    assert worst_d <= bound, f"{what}: max |logit - plain| = {worst_d:.3e} at request/position {where} (bound {bound:.3e})"


@pytest.mark.parametrize("name,dtype,page", [("F", "float32", None), ("F", "bfloat16", None), ("F", "bfloat16", 64),
                                             ("R", "float32", None), ("R", "bfloat16", None), ("R", "bfloat16", 64)])
def test_replay_long_portions_beside_decoding_requests(name, dtype, page, tiny_folders, plain_models, real_size_model,
                                                      tmp_path):
    """Portions of 129 to 1024 tokens beside three requests that decode, in one step: the products with tokens on
    the tile's rows and the q,k,v epilogue over rows of different requests, the prompt attention and the decode
    attention in the same step."""
    if name == "R":
        folder, cfg, t = real_size_model
    else:
        folder, (cfg, t) = tiny_folders[name], plain_models[name]
    dec_lens, big_portions = SERVING[name]
    decoders = {f"d{i}": random_ids(cfg["vocab_size"], n, 300 + i) for i, n in enumerate(dec_lens)}
    bigs = [(f"big{i}", random_ids(cfg["vocab_size"], sum(por), 400 + i), por) for i, por in enumerate(big_portions)]
    tr = Trace()
    play_serving_steps(tr, decoders, bigs)
    got = run_trace(folder, dtype, tr, str(tmp_path), tr.live_peak, page)
    reqs = {**decoders, **{n: ids for n, ids, _ in bigs}}
    check_against_plain(got, reqs, cfg, t, dtype, "long portions beside decoding")


def play_many_decoding(tr: Trace, reqs: dict[str, list[int]], n_decode: int, per_step: int = 8):
    names = list(reqs)
    for i in range(0, len(names), per_step):
        tr.step({n: reqs[n][:len(reqs[n]) - n_decode] for n in names[i:i + per_step]})
    for k in range(n_decode, 0, -1):
        tr.step({n: reqs[n][len(reqs[n]) - k:len(reqs[n]) - k + 1] for n in names}, end=names if k == 1 else [])


@pytest.mark.parametrize("name,dtype,live", [("F", "bfloat16", 9), ("F", "bfloat16", 33), ("F", "bfloat16", 65),
                                             ("F", "float32", 33), ("D", "bfloat16", 65), ("R", "bfloat16", 9),
                                             ("R", "bfloat16", 65)])
def test_replay_many_requests_decoding_together(name, dtype, live, tiny_folders, plain_models, real_size_model, tmp_path):
    """Decode steps of 9, 33 and 65 live requests (the captured graphs' buckets of 16, 64 and 128 rows, the
    products' tiles of 16 to 128 tokens, the attention with and without a split of the context)."""
    if name == "R":
        folder, cfg, t = real_size_model
    else:
        folder, (cfg, t) = tiny_folders[name], plain_models[name]
    rng = random.Random(live)
    reqs = {f"q{i}": random_ids(cfg["vocab_size"], rng.choice([7, 12, 20, 33, 49, 64, 65, 90]) if name != "R"
                                else rng.choice([6, 9, 17, 30]), 500 + i) for i in range(live)}
    tr = Trace()
    play_many_decoding(tr, reqs, n_decode=4)
    got = run_trace(folder, dtype, tr, str(tmp_path), tr.live_peak, None, max_requests=live)
    check_against_plain(got, reqs, cfg, t, dtype, f"{live} requests decoding")
