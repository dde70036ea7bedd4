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
def layer_matrix_params(cfg) -> int:
    H, I = cfg.hidden_size, cfg.intermediate_size
    return H * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * H + 3 * H * I


def kv_bytes_per_token(cfg, num_layers: int, itemsize: int = 2) -> int:
    return num_layers * 2 * cfg.kv_size * itemsize


def decode_step_bytes(cfg, num_layers: int, batch: int, context: int, itemsize: int = 2) -> int:
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    weights = (num_layers * (layer_matrix_params(cfg) + 2 * cfg.hidden_size + 2 * cfg.head_dim) + cfg.hidden_size
               + cfg.vocab_size * cfg.hidden_size) * itemsize
    return weights + batch * context * kv_bytes_per_token(cfg, num_layers, itemsize)


def prefill_flops(cfg, num_layers: int, tokens: int, logit_rows: int = 1) -> float:
    matmul = 2.0 * tokens * num_layers * layer_matrix_params(cfg) + 2.0 * logit_rows * cfg.vocab_size * cfg.hidden_size
    attention = num_layers * 4.0 * cfg.num_attention_heads * cfg.head_dim * tokens * (tokens + 1) / 2
    return matmul + attention


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
    """W untimed then K timed decode steps of the live requests ``names``; tokens stay on the device."""
    B = len(names)
    dev = runner.rt.device
    tokens = torch.full((B,), 11, dtype=torch.int32, device=dev)
    entries = [StepEntry(n, [0], (0,)) for n in names]

    def one():
        logits = runner.step(entries, device_tokens=tokens)
        ops.argmax(logits, tokens)

    for _ in range(warmup):
        one()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    launches0 = ops.LAUNCHES + getattr(runner, "graph_launches", 0)
    start.record()
    for _ in range(steps):
        one()
    end.record()
    torch.cuda.synchronize(dev)
    ms = start.elapsed_time(end) / steps
    launches = ops.LAUNCHES + getattr(runner, "graph_launches", 0) - launches0
    return {"ms_per_step": ms, "tokens_per_s": B * 1000.0 / ms, "launches": launches, "batch": B,
            "context_end": runner.manager.lengths[names[0]]}


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
