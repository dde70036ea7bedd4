"""Measurement of decode and prefill throughput, device-timed.

The protocol follows the reference's ``bench_decode`` (acvram/bench.py:311-503):
warm-up first, synthetic token ids, what was actually processed is what is
reported, and a number whose preconditions failed is refused rather than
published.  Times are CUDA events on the launching stream with a synchronize on
both sides; the decode loop keeps its sampled tokens on the device, so the timed
region holds no host round trip (the end-to-end number, with one, is measured
through ``Engine.step``).
"""

from __future__ import annotations

import statistics
import subprocess
import threading
import time

import torch

from .engine.batch import StepEntry
from .kernels import ops


# --------------------------------------------------------------------------- arithmetic of a step
# What a step has to read and compute is asked of the model (``DecoderModel.step_cost``: every scheduled part reports
# its own weights, products, mixing and cache reads), so the figures follow the plan that runs, whatever the architecture.
def decode_step_bytes(model, batch: int, context: int) -> int:
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    cost = model.step_cost([1] * batch, [context] * batch, batch)
    return cost["weight_bytes"] + cost["cache_bytes"]


def prefill_flops(model, tokens: int, logit_rows: int = 1) -> float:
    return model.step_cost([tokens], [tokens], logit_rows)["flops"]


class Refused(RuntimeError):
    """A measurement whose preconditions failed: its number is not published (acvram/bench.py:426-447)."""


# --------------------------------------------------------------------------- clocks during the timed region
class ClockSampler:
    """Samples nvidia-smi every 200 ms in the background (reads only; changes nothing)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0) -> None:
        self.index = index
        self.lines: list[str] = []
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def __exit__(self, *exc):
        if self.proc is not None:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val == "Active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "power_w": statistics.median(power), "samples": len(sm)}


# --------------------------------------------------------------------------- workloads
def synthetic_ids(vocab: int, n: int, k: int) -> list[int]:
    """The reference's synthetic prompt, distinct for each k (acvram/bench.py:375-377)."""
    return [(k * 104729 + i * 7919) % max(1, vocab - 100) + 10 for i in range(n)]


def fill_contexts(runner, names: list, context: int, chunk: int = 2048) -> None:
    """Give each named request a context of ``context`` synthetic tokens (prefilled in portions)."""
    vocab = runner.model.plan.vocab_size
    for k, name in enumerate(names):
        ids = synthetic_ids(vocab, context, k)
        for pos in range(0, context, chunk):
            runner.step([StepEntry(name, ids[pos:pos + chunk], ())])


def time_decode(runner, names: list, steps: int, warmup: int) -> dict:
    """W untimed then K timed decode steps of the live requests ``names``; tokens stay on the device.

    Refused (``Refused``) when a timed step did not replay a captured graph although graphs are on, when a kernel
    gave up a bounded wait, or when the requests did not all advance by exactly K + W tokens."""
    B = len(names)
    dev = runner.rt.device
    tokens = torch.full((B,), 11, dtype=torch.int32, device=dev)
    entries = [StepEntry(n, [0], (0,)) for n in names]
    before = [runner.manager.lengths[n] for n in names]

    def one():
        logits = runner.step(entries, device_tokens=tokens)
        ops.argmax(logits, tokens)

    for _ in range(warmup):
        one()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    launches0 = ops.LAUNCHES + getattr(runner, "graph_launches", 0)
    replays0 = runner.graphs.replays if runner.graphs is not None else 0
    start.record()
    for _ in range(steps):
        one()
    end.record()
    torch.cuda.synchronize(dev)
    ms = start.elapsed_time(end) / steps
    launches = ops.LAUNCHES + getattr(runner, "graph_launches", 0) - launches0
    code = ops.gemm_status()
    if code:
        ops.reset_after_failure()
        raise Refused(f"a kernel gave up a bounded wait during the timed steps (status {code})")
    if runner.graphs is not None and runner.graphs.disabled_reason is None and runner.graphs.replays - replays0 != steps:
        raise Refused(f"{steps - (runner.graphs.replays - replays0)} of {steps} timed steps did not replay a captured graph")
    if [runner.manager.lengths[n] - b for n, b in zip(names, before)] != [steps + warmup] * B:
        raise Refused("the requests did not all advance by one token per step")
    return {"ms_per_step": ms, "tokens_per_s": B * 1000.0 / ms, "launches": launches, "batch": B,
            "context_end": runner.manager.lengths[names[0]]}


def time_mixed(runner, names: list, portion: int, prompt_len: int, steps: int, warmup: int) -> dict:
    """Steps that serving makes under load: every live request of ``names`` decodes one token beside a portion of
    ``portion`` tokens of another request's prompt (prompts of ``prompt_len`` tokens, one after the other; a prompt
    that is through gives its pages to the next).  Returns ms per step and tokens per second (all tokens of a step)."""
    B = len(names)
    dev = runner.rt.device
    vocab = runner.model.plan.vocab_size
    tokens = torch.full((B,), 11, dtype=torch.int32, device=dev)
    state = {"k": 0, "pos": 0, "ids": synthetic_ids(vocab, prompt_len, 5000)}

    def one():
        name = f"mixed-prompt-{state['k']}"
        ids = state["ids"][state["pos"]:state["pos"] + portion]
        last = state["pos"] + len(ids) >= prompt_len
        entries = [StepEntry(n, [11], (0,)) for n in names] + [StepEntry(name, ids, (len(ids) - 1,) if last else ())]
        logits = runner.step(entries)
        ops.argmax(logits[:B], tokens)
        state["pos"] += len(ids)
        if last:
            runner.release(name)
            state.update(k=state["k"] + 1, pos=0, ids=synthetic_ids(vocab, prompt_len, 5001 + state["k"]))

    for _ in range(warmup):
        one()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    start.record()
    for _ in range(steps):
        one()
    end.record()
    torch.cuda.synchronize(dev)
    name = f"mixed-prompt-{state['k']}"
    if name in runner.manager.lengths:
        runner.release(name)
    code = ops.gemm_status()
    if code:
        ops.reset_after_failure()
        raise Refused(f"a kernel gave up a bounded wait during the timed steps (status {code})")
    ms = start.elapsed_time(end) / steps
    return {"ms_per_step": ms, "tokens_per_s": (B + portion) * 1000.0 / ms, "decode_tokens_per_s": B * 1000.0 / ms}


def time_prefill(runner, tokens: int, reps: int = 3, warmup: int = 1) -> dict:
    """One prompt of ``tokens`` tokens in one step, a new request and new ids each time."""
    vocab = runner.model.plan.vocab_size
    times = []
    for k in range(warmup + reps):
        ids = synthetic_ids(vocab, tokens, 1000 + k)
        name = f"prefill-{k}"
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry(name, ids, (tokens - 1,))])
        end.record()
        torch.cuda.synchronize()
        runner.release(name)
        if k >= warmup:
            times.append(start.elapsed_time(end))
    code = ops.gemm_status()
    if code:
        ops.reset_after_failure()
        raise Refused(f"a kernel gave up a bounded wait during the timed steps (status {code})")
    ms = statistics.median(times)
    return {"ms": ms, "tokens": tokens, "tokens_per_s": tokens * 1000.0 / ms, "spread_ms": max(times) - min(times)}


def bench_decode(model, random_weights=False, seed=0, dtype="bfloat16", batches=(1,), context=128, n_tokens=256,
                 device="cuda:0", cuda_graphs=True, repetitions=3, prefill=0) -> dict:
    """``acvram bench --what decode``: median decode tokens/s for each batch size, with the spread; with
    ``prefill`` > 0 also the tokens/s of one prompt of that many tokens computed in one step."""
    from .engine import Engine
    need = max(max(batches) * (context + n_tokens + 64), prefill + 64)
    eng = Engine(model, dtype, max_batch_size=max(batches), max_model_len=max(context + n_tokens, prefill) + 64,
                 random_weights=random_weights, seed=seed, device=device, enable_cuda_graphs=cuda_graphs,
                 page_size=64, num_pages=need // 64 + 2 * max(batches), enable_prefix_cache=False)
    out = {"model": str(model), "dtype": dtype, "context": context, "tokens": n_tokens}
    for b in batches:
        rates = []
        for rep in range(repetitions):
            names = [f"b{b}-{rep}-{i}" for i in range(b)]
            fill_contexts(eng.runner, names, context)
            r = time_decode(eng.runner, names, n_tokens, 3)
            rates.append(r["tokens_per_s"])
            for n in names:
                eng.runner.release(n)
        out[f"decode_b{b}"] = {"tokens_per_s": statistics.median(rates), "spread": max(rates) - min(rates),
                               "runs": rates}
    if prefill > 0:
        if prefill > eng.max_model_len:
            raise ValueError(f"a prefill of {prefill} tokens does not fit the model's {eng.max_model_len} positions")
        out["prefill"] = time_prefill(eng.runner, prefill, reps=3, warmup=1)
    return out
