"""CUDA-graph replay of the decode step.

A step in which every request brings one token has the same launches whatever the
requests are, once the batch is padded to a bucket and the longest context is
rounded up to a bucket (it decides how the attention splits its work); the whole
model step is then captured once per (batch bucket, context bucket) and replayed, which removes the per-launch cost of some three hundred
launches a step.  The idea, buckets and padding rows follow the reference's
``GraphRunner`` (acvram/engine/graphs.py:8-22, 49-72; padding rows carry a context
length of 0 and write nothing, acvram/engine/graphs.py:14-17).  Each graph owns a
static metadata buffer; a step copies what changes from step to step there (tokens,
positions, context lengths, the requests' rows of the block tables, which stay on
the device, and the few table entries that changed) and replays.
"""

from __future__ import annotations

import gc

import torch

from ..kernels import ops

BATCH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)
MIN_TABLE_WIDTH = 8
MAX_GRAPHS = 64   # the reference keeps at most 64 as well


def batch_bucket(n: int) -> int:
    for b in BATCH_BUCKETS:
        if n <= b:
            return b
    return 0


def width_bucket(pages: int) -> int:
    w = MIN_TABLE_WIDTH
    while w < pages:
        w *= 2
    return w


class DecodeGraphs:
    def __init__(self, runner) -> None:
        self.runner = runner
        self.graphs: dict[tuple[int, int], dict] = {}
        self.replays = 0
        self.launches = 0       # kernels of this package run through replays
        self.refused = 0        # decode steps that ran without a graph because the table of graphs was full
        self.disabled_reason: str | None = None
        # a part whose forward reads device memory on the host (a toy that loops over requests in Python, say)
        # cannot be captured; everything else can, state of fixed size included (its slots travel with the step)
        blocked = runner.model.uncapturable_parts() if hasattr(runner.model, "uncapturable_parts") else []
        if blocked:
            self.disabled_reason = "parts that cannot run in a CUDA graph: " + ", ".join(blocked)

    def usable(self, entries) -> bool:
        return (self.disabled_reason is None and all(len(e.tokens) == 1 for e in entries)
                and batch_bucket(len(entries)) > 0)

    def run(self, entries, starts, device_tokens=None) -> torch.Tensor:
        """Logits [len(entries), vocab] of a decode step, through a captured graph."""
        r = self.runner
        m = r.manager
        padded = batch_bucket(len(entries))
        pages = max(g.pages_for(s + 1) for g in m.paged_groups for s in starts)
        width = width_bucket(pages)
        key = (padded, width)
        slot = self.graphs.get(key)
        if slot is None:
            if len(self.graphs) >= MAX_GRAPHS:
                self.refused += 1
                return None
            slot = self._capture(key, entries, starts, device_tokens)
        else:
            ctx = r.builder.build_decode(entries, starts, padded, width * m.page_size, slot["dev"])
            if device_tokens is not None:
                ctx.tokens[:len(entries)].copy_(device_tokens)
            slot["graph"].replay()
        self.replays += 1
        self.launches += slot["kernels"]
        return slot["logits"][:len(entries)]

    def _capture(self, key, entries, starts, device_tokens):
        r = self.runner
        padded, width = key
        _, _, total = r.builder.decode_layout(padded)
        dev = torch.empty(total, dtype=torch.int32, device=r.rt.device)
        # the launch shapes (how the attention splits the context) follow the bucket's longest context,
        # width * page_size, whatever the requests of this step hold
        ctx = r.builder.build_decode(entries, starts, padded, width * r.manager.page_size, dev, first=True)
        if device_tokens is not None:
            ctx.tokens[:len(entries)].copy_(device_tokens)
        # This step itself runs eagerly (scratch buffers reach their size on the way) and its logits are the step's
        # answer; the capture below records the same launches without running them.  Replaying the new graph for this
        # step as well would run the step twice, which a mixer that adds to a state of its own must not see.
        eager_logits = r.model.forward(ctx, r.storage)
        torch.cuda.synchronize(r.rt.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        # While a stream is being captured, CUDA by default refuses calls it counts as unsafe from anywhere in the
        # process (freeing pinned memory, destroying another graph, querying an event) and the capture is lost.
        # The garbage collector makes such calls when it finalises objects of an engine that is no longer used; seen
        # as a capture that failed now and then in a process that had built many engines.  None of them touches the
        # capturing stream, so the capture runs in relaxed mode, and the collector rests while it lasts.
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(graph, capture_error_mode="relaxed"):
                logits = r.model.forward(ctx, r.storage)
        finally:
            if gc_was_on:
                gc.enable()
        kernels = ops.LAUNCHES - before
        logits.copy_(eager_logits)
        slot = {"graph": graph, "dev": dev, "ctx": ctx, "logits": logits, "kernels": kernels}
        self.graphs[key] = slot
        return slot
