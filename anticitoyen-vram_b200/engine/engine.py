"""The Python entry point: ``Engine(...).generate(...)``.

Names and meanings follow the reference's ``Engine`` (acvram/engine/runner.py:689-694,
2680-2689): ``add_request``, ``step``, ``generate``, ``abort``, ``idle``, ``stats``;
``max_batch_size`` and ``max_model_len`` as there.  Where the reference takes a
converted checkpoint, this engine takes a model folder (config.json and
safetensors) or a typed configuration with ``random_weights``.
"""

from __future__ import annotations

import itertools
import time
from dataclasses import dataclass, field
from typing import Hashable, Iterator, Optional, Sequence

import torch

from ..kernels import ops
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, StepPlan
from .text import cut_at_stop, text_delta


@dataclass
class GenerationOutput:
    """What a step delivers for a request (acvram/engine/runner.py:203-217)."""

    sequence_id: int
    request_id: Hashable
    token_ids: list[int]
    text_delta: str = ""
    finished: bool = False
    finish_reason: Optional[str] = None
    prompt_tokens: int = 0
    completion_tokens: int = 0
    logprob: Optional[float] = None          # of the delivered token, for requests with ``logprobs`` set
    top_logprobs: Optional[list] = None      # [(token id, log probability)], most probable first, ``logprobs`` of them
    cumulative_logprob: Optional[float] = None
    error: Optional[str] = None              # with finish_reason "error": what went wrong in the request's step


@dataclass
class EngineStats:
    """Counters with cumulative seconds, not only rates (acvram/engine/runner.py:321-363)."""

    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    preempted: int = 0
    refused: int = 0
    truncated: int = 0
    reused_tokens: int = 0       # prompt tokens taken over from published pages instead of being computed
    failed_steps: int = 0        # steps that raised or whose kernels reported a wait that ran out
    failed_requests: int = 0     # requests ended with finish_reason "error" by such steps
    extra: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        d = {k: v for k, v in self.__dict__.items() if k != "extra"}
        d.update(self.extra)
        return d


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


@dataclass
class _Flight:
    """A step that has been launched and not yet read."""
    plan: StepPlan
    rows: list                 # the requests that get a token, in the order of ``tokens``
    tokens: torch.Tensor | None
    logprobs: torch.Tensor | None
    top: tuple | None          # (ids [rows, k], log probabilities [rows, k]) on the device, when a request asks for them
    host: torch.Tensor | None  # pinned copy of ``tokens``, valid after ``event``
    status: torch.Tensor       # pinned copy of the kernels' status word after the step, valid after ``event``
    event: torch.cuda.Event
    t0: float
    decode: int
    prefill: int


class Engine:
    def __init__(self, model, dtype="bfloat16", *, max_batch_size: int = 16, max_model_len: int = 8192,
                 page_size: int = 64, num_pages: int | None = None, token_budget: int = 2048,
                 random_weights: bool = False, seed: int = 0, device: str = "cuda:0",
                 enable_cuda_graphs: bool = True, run_ahead: bool = True, enable_prefix_cache: bool = True,
                 tokenizer=None, fuse_decode_layers: bool = False) -> None:
        """``model``: a folder with config.json and model.safetensors, or (with
        ``random_weights``) a typed configuration or a folder whose config.json alone is read.
        ``tokenizer``: anything with ``decode(ids) -> str``; with one, outputs carry the text that their tokens
        add (``text_delta``) and ``SamplingParams.stop`` strings end a request.
        ``enable_prefix_cache`` (the reference's name and default, acvram/engine/runner.py:689-694): the full
        pages of a finished request stay known, and a later request that begins the same way takes them over.
        ``fuse_decode_layers``: steps of up to 16 decoding requests run each layer as one persistent kernel instead
        of seven launches (slower on a B200 at the sizes measured; kept as a choice)."""
        from ..config import load_config
        from ..models import build_from_folder, build_random

        run_dtype = _DTYPES[dtype]
        if not torch.cuda.is_available():
            raise RuntimeError("acvram_b200 needs a CUDA device: its kernels have no CPU path")
        if hasattr(model, "plan") and hasattr(model, "forward"):     # a model already built and loaded
            self.model, self.config = model, None
        elif random_weights:
            config = load_config(model) if isinstance(model, (str, bytes)) or hasattr(model, "__fspath__") else model
            self.model = build_random(config, seed, run_dtype, device)
            self.config = config
        else:
            self.config, self.model = build_from_folder(model, run_dtype, device)
        plan = self.model.plan
        for block in getattr(self.model, "blocks", ()):
            if hasattr(block, "fuse_decode"):
                block.fuse_decode = bool(fuse_decode_layers)
        self.max_model_len = min(max_model_len, plan.max_positions)
        self.page_size = page_size
        if num_pages is None:
            num_pages = self._default_pages(max_batch_size, device)
        self.runner = ModelRunner(self.model, page_size, num_pages, max_batch_size, enable_prefix_cache,
                                  max_len=self.max_model_len)
        self.scheduler = Scheduler(self.runner.manager, max_batch_size, token_budget, self.max_model_len)
        self.sampler = Sampler(device)
        self.tokenizer = tokenizer
        self.seed = seed
        self.stats = EngineStats()
        self.enable_cuda_graphs = enable_cuda_graphs and run_dtype == torch.bfloat16
        if self.enable_cuda_graphs:
            self.runner.enable_graphs()
        self._ids = itertools.count()
        # one step ahead (see ``step``): the launched, unread step and two pinned buffers for sampled tokens
        self.pipeline = run_ahead
        self._flight: _Flight | None = None
        self._pinned = [torch.empty(max_batch_size, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._pinned_status = [torch.zeros(1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._pinned_turn = 0
        self._status = ops.status_word(self.model.rt.device)
        self._open: list[StepPlan] = []      # plans whose steps are launched or being launched, not yet committed
        self._early: list[GenerationOutput] = []
        self.last_error: str | None = None
        self._requests: dict[Hashable, Request] = {}
        self._seq_ids: dict[Hashable, int] = {}

    def _default_pages(self, max_batch_size: int, device) -> int:
        """Pages for max_batch_size requests of max_model_len tokens, within 85 % of the free memory."""
        per_page = state_bytes = 0
        for need in self.model.cache_plan().needs:
            if need is not None and need.kind == "paged":
                per_page += 2 * need.num_kv_heads * need.head_dim * self.page_size * self.model.rt.dtype.itemsize
            elif need is not None:       # state of fixed size: a slot for each request (and one for nobody)
                n = 1
                for d in need.shape:
                    n *= d
                state_bytes += n * getattr(torch, need.dtype).itemsize * (max_batch_size + 1)
        want = max_batch_size * ((self.max_model_len + self.page_size - 1) // self.page_size)
        free, _ = torch.cuda.mem_get_info(torch.device(device))
        fit = int(max(0, free * 0.85 - state_bytes) // max(per_page, 1))
        return max(1, min(want, fit))

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt_ids: Sequence[int], params: SamplingParams | None = None,
                    request_id: Hashable | None = None) -> Hashable:
        params = params or SamplingParams()
        n = next(self._ids)
        request_id = request_id if request_id is not None else f"req-{n}"
        seed = params.seed if params.seed is not None else (self.seed * 1000003 + n) & 0x7FFFFFFFFFFFFFFF
        req = Request(request_id, list(prompt_ids), params, seed)
        vocab = self.model.plan.vocab_size
        if any(not 0 <= t < vocab for t in req.prompt):
            raise ValueError(f"prompt token outside the vocabulary of {vocab}")
        self.scheduler.add(req)
        self._requests[request_id] = req
        self._seq_ids[request_id] = n
        return request_id

    def abort(self, request_id: Hashable) -> None:
        self.scheduler.abort(request_id)
        self._requests.pop(request_id, None)

    @property
    def idle(self) -> bool:
        return self.scheduler.idle and self._flight is None

    # ------------------------------------------------------------------ one step
    def step(self) -> list[GenerationOutput]:
        """Run one step and deliver what is known by its end.

        While every running request decodes and nobody waits, the engine works one step ahead: it launches
        step k+1 (whose tokens it feeds on the device) before it reads step k's tokens, so that the host's
        share of a step (planning, the batch's tables, the launch, reading the tokens) falls into the time
        the device computes.  A call then delivers the tokens of the step launched one call earlier; the
        first such call delivers nothing.  ``idle`` stays false until the last launched step is delivered.

        A step that raises, or whose kernels report a bounded wait that ran out (their status word, read
        with the step's tokens), does not stop the engine: the requests of that step end with
        ``finish_reason="error"``, their pages go back without becoming known to later requests, and
        requests that wait or were not part of the step are served as before
        (acvram/engine/runner.py:1329-1338)."""
        self._early = []
        try:
            return self._step()
        except Exception as exc:          # not BaseException: an interrupt still ends the caller's loop
            return self._fail(exc)

    def _step(self) -> list[GenerationOutput]:
        flight, self._flight = self._flight, None
        if flight is not None:
            ahead = self.scheduler.schedule_ahead(flight.plan) if self._can_run_ahead(flight) else None
            if ahead is not None:
                self._open.append(ahead)
                self._flight = self._launch(ahead, flight)
            return self._complete(flight)
        plan = self.scheduler.schedule()
        self._open.append(plan)
        outputs = self._early = [self._output(r, []) for r in plan.refused + plan.truncated]
        self.stats.preempted += len(plan.preempted)
        self.stats.refused += len(plan.refused)
        self.stats.truncated += len(plan.truncated)
        self.stats.reused_tokens = self.scheduler.counters["reused_tokens"]
        if not plan.entries:
            self._open.remove(plan)
            return outputs
        flight = self._launch(plan, None)
        if self.pipeline and self._can_run_ahead(flight) and self.scheduler.schedule_ahead_possible(plan):
            self._flight = flight          # delivered by the next call, which launches the step after it first
            return outputs
        return outputs + self._complete(flight)

    def _can_run_ahead(self, flight: "_Flight") -> bool:
        return (self.pipeline and flight.logprobs is None and not flight.prefill
                and all(not r.params.penalised for r in flight.rows))

    def _launch(self, plan: StepPlan, after: "_Flight | None") -> "_Flight":
        """Enqueue the step, its sampling and the copy of the sampled tokens to pinned memory; no wait.
        ``after``: the step before, still unread; its sampled tokens are this step's inputs, on the device."""
        t0 = time.perf_counter()
        device_tokens = None
        lag = 0
        if after is not None:
            lag = 1
            pos = {id(r): i for i, r in enumerate(after.rows)}
            idx = [pos[id(e.request)] for e in plan.entries]
            device_tokens = after.tokens
            if idx != list(range(len(after.rows))):
                # some requests ended with the step before: the others' tokens, gathered run by run with plain
                # device copies (no kernel of another library on the step's path)
                device_tokens = torch.empty(len(idx), dtype=after.tokens.dtype, device=after.tokens.device)
                a = 0
                while a < len(idx):
                    b = a + 1
                    while b < len(idx) and idx[b] == idx[b - 1] + 1:
                        b += 1
                    device_tokens[a:b].copy_(after.tokens[idx[a]:idx[a] + (b - a)])
                    a = b
            entries = [StepEntry(e.request.request_id, [0], (0,)) for e in plan.entries]
        else:
            entries = [StepEntry(e.request.request_id, e.request.token_slice(e.start, e.count),
                                 (e.count - 1,) if e.samples else ()) for e in plan.entries]
        logits = self.runner.step(entries, device_tokens=device_tokens)
        rows = [e.request for e in plan.entries if e.samples]
        tokens = logprobs = host = top = None
        event = torch.cuda.Event()
        if rows:
            want_lp = any(r.params.logprobs is not None for r in rows)
            # the k most probable tokens are read from the logits as the model gave them, before penalties and
            # temperature, one k for the whole step (the largest asked for), as the reference does
            # (acvram/engine/runner.py:2625-2640)
            k = max((int(r.params.logprobs or 0) for r in rows), default=0)
            if k > 0:
                top = ops.top_logprobs(logits, min(k, 64, logits.shape[1]))
            tokens, logprobs = self.sampler(
                logits, [r.params for r in rows], [r.tokens if r.params.penalised else () for r in rows],
                [r.seed for r in rows], [len(r.output) + lag for r in rows], want_lp)
            host = self._pinned[self._pinned_turn][:len(rows)]
            host.copy_(tokens, non_blocking=True)
        status = self._pinned_status[self._pinned_turn]
        status.copy_(self._status, non_blocking=True)
        self._pinned_turn ^= 1
        event.record()
        decode = sum(1 for e in plan.entries if e.count == 1 and e.start > 0)
        return _Flight(plan, rows, tokens, logprobs, top, host, status, event, t0, decode, plan.num_tokens - decode)

    def _complete(self, f: "_Flight") -> list[GenerationOutput]:
        """Wait for the step's tokens (the step's one wait for the device), record them, make the outputs."""
        f.event.synchronize()
        code = int(f.status[0])
        if code:
            raise ops.KernelError(f"a kernel of the step gave up a bounded wait (status {code}): its results are not used")
        sampled = f.host.tolist() if f.host is not None else []
        logprobs = f.logprobs.tolist() if f.logprobs is not None else None
        top = (f.top[0].tolist(), f.top[1].tolist()) if f.top is not None else None
        dt = time.perf_counter() - f.t0
        before = {id(r): len(r.output) for r in f.rows}
        touched = self.scheduler.commit(f.plan, sampled, self.model.plan.eos_token_ids)
        self._open.remove(f.plan)
        row_of = {id(r): i for i, r in enumerate(f.rows)}
        outputs = []
        for r in touched:
            new = r.output[before[id(r)]:]
            lp = tops = None
            if logprobs is not None and new and r.params.logprobs is not None:
                lp = logprobs[row_of[id(r)]]
                r.logprob_sum += lp
                if top is not None and r.params.logprobs > 0:
                    i, n = row_of[id(r)], int(r.params.logprobs)
                    tops = [(t, p) for t, p in zip(top[0][i][:n], top[1][i][:n]) if t >= 0]
            outputs.append(self._output(r, new, lp, tops, self._text(r) if self.tokenizer is not None else ""))
        self.stats.steps += 1
        self.stats.decode_tokens += f.decode
        self.stats.prefill_tokens += f.prefill
        if f.prefill:
            self.stats.prefill_seconds += dt
        else:
            self.stats.decode_seconds += dt
        return outputs

    def _fail(self, exc: Exception, always: bool = False) -> list[GenerationOutput]:
        """End the requests of every step that is launched or was being launched and not committed.

        The device is waited for first (a step launched ahead may still run and write pages that are about to go
        back); if that wait fails too, the CUDA context is lost and the first exception is raised again.  An
        exception from outside a step (every plan is committed: a tokenizer that raised, say) is not the
        engine's to absorb and is raised again as well."""
        plans, self._open = self._open, []
        self._flight = None
        if not plans and not always:
            raise exc
        try:
            torch.cuda.synchronize(self.model.rt.device)
            ops.reset_after_failure()
            self.runner.manager.resync()      # the step's changes of the block tables may not have reached the device
        except Exception:
            raise exc
        text = f"{type(exc).__name__}: {exc}"
        self.last_error = text
        failed = self.scheduler.fail([e.request for plan in plans for e in plan.entries])
        self.stats.failed_steps += 1
        self.stats.failed_requests += len(failed)
        outputs = list(self._early)
        for r in failed:
            out = self._output(r, [])
            out.error = text
            outputs.append(out)
        return outputs

    def fail_step(self, reason: str = "a caller gave the step up") -> list[Hashable]:
        """What the reference's ``echec_du_pas`` does for its server (acvram/engine/runner.py:1329-1338): end the
        requests of the steps in flight with ``"error"``, give their pages back unpublished; returns their ids."""
        self._early = []
        return [o.request_id for o in self._fail(RuntimeError(reason), always=True) if o.finish_reason == "error"]

    def _text(self, r: Request) -> str:
        """The text that the request's new tokens add; ends the request where a stop string begins
        (acvram/engine/runner.py:2550-2557: the string itself is not delivered)."""
        delta, r.text_tokens = text_delta(self.tokenizer, r.output, r.text_tokens, final=r.finished)
        r.text += delta
        if delta and r.params.stop and (not r.finished or r.finish_reason == "length"):
            kept, hit = cut_at_stop(r.text, delta, r.params.stop)
            if hit:
                r.text = r.text[:len(r.text) - len(delta) + len(kept)]
                delta = kept
                if r.finished:
                    r.finish_reason = "stop"
                else:
                    self.scheduler.finish(r, "stop")
        return delta

    def _output(self, r: Request, new: list[int], logprob: float | None = None, top: list | None = None,
                text: str = "") -> GenerationOutput:
        if r.finished:
            self._requests.pop(r.request_id, None)
        return GenerationOutput(self._seq_ids.get(r.request_id, -1), r.request_id, list(new), text, r.finished,
                                r.finish_reason, len(r.prompt), len(r.output), logprob, top,
                                r.logprob_sum if r.params.logprobs is not None else None)

    # ------------------------------------------------------------------ generation
    def generate(self, prompt_ids: Sequence[int], params: SamplingParams | None = None) -> Iterator[GenerationOutput]:
        """One request to its end, blocking; yields what each step delivers for it
        (acvram/engine/runner.py:2680-2689)."""
        rid = self.add_request(prompt_ids, params)
        while True:
            done = False
            for out in self.step():
                if out.request_id == rid:
                    yield out
                    done = done or out.finished
            if done or self.idle:
                return

    def generate_batch(self, prompts: Sequence[Sequence[int]], params: SamplingParams | Sequence[SamplingParams] | None = None
                       ) -> list[list[int]]:
        """Several requests together, to their ends; the generated ids of each, in order."""
        if params is None or isinstance(params, SamplingParams):
            params = [params] * len(prompts)
        ids = [self.add_request(p, sp) for p, sp in zip(prompts, params)]
        got: dict[Hashable, list[int]] = {i: [] for i in ids}
        while not self.idle:
            for out in self.step():
                if out.request_id in got:
                    got[out.request_id].extend(out.token_ids)
        return [got[i] for i in ids]
