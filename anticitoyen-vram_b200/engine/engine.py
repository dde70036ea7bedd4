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

from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Request, Scheduler, StepPlan


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
    logprob: float = 0.0
    top_logprobs: Optional[list] = None


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
    extra: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        d = {k: v for k, v in self.__dict__.items() if k != "extra"}
        d.update(self.extra)
        return d


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


class Engine:
    def __init__(self, model, dtype="bfloat16", *, max_batch_size: int = 16, max_model_len: int = 8192,
                 page_size: int = 64, num_pages: int | None = None, token_budget: int = 2048,
                 random_weights: bool = False, seed: int = 0, device: str = "cuda:0",
                 enable_cuda_graphs: bool = True, tokenizer=None) -> None:
        """``model``: a folder with config.json and model.safetensors, or (with
        ``random_weights``) a typed configuration or a folder whose config.json alone is read."""
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
        self.max_model_len = min(max_model_len, plan.max_positions)
        self.page_size = page_size
        if num_pages is None:
            num_pages = self._default_pages(max_batch_size, device)
        self.runner = ModelRunner(self.model, page_size, num_pages, max_batch_size)
        self.scheduler = Scheduler(self.runner.manager, max_batch_size, token_budget, self.max_model_len)
        self.sampler = Sampler(device)
        self.tokenizer = tokenizer
        self.seed = seed
        self.stats = EngineStats()
        self.enable_cuda_graphs = enable_cuda_graphs and run_dtype == torch.bfloat16
        if self.enable_cuda_graphs:
            self.runner.enable_graphs()
        self._ids = itertools.count()
        self._requests: dict[Hashable, Request] = {}
        self._seq_ids: dict[Hashable, int] = {}

    def _default_pages(self, max_batch_size: int, device) -> int:
        """Pages for max_batch_size requests of max_model_len tokens, within 85 % of the free memory."""
        per_page = 0
        for need in self.model.cache_plan().needs:
            if need is not None and need.kind == "paged":
                per_page += 2 * need.num_kv_heads * need.head_dim * self.page_size * self.model.rt.dtype.itemsize
        want = max_batch_size * ((self.max_model_len + self.page_size - 1) // self.page_size)
        free, _ = torch.cuda.mem_get_info(torch.device(device))
        fit = int(free * 0.85 // max(per_page, 1))
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
        return self.scheduler.idle

    # ------------------------------------------------------------------ one step
    def step(self) -> list[GenerationOutput]:
        plan = self.scheduler.schedule()
        outputs = [self._output(r, []) for r in plan.refused + plan.truncated]
        self.stats.preempted += len(plan.preempted)
        self.stats.refused += len(plan.refused)
        self.stats.truncated += len(plan.truncated)
        if not plan.entries:
            return outputs
        t0 = time.perf_counter()
        entries = [StepEntry(e.request.request_id, e.request.tokens[e.start:e.start + e.count],
                             (e.count - 1,) if e.samples else ()) for e in plan.entries]
        logits = self.runner.step(entries)
        rows = [e.request for e in plan.entries if e.samples]
        sampled: list[int] = []
        logprobs = None
        if rows:
            want_lp = any(r.params.logprobs is not None for r in rows)
            tokens, logprobs = self.sampler(
                logits, [r.params for r in rows], [r.tokens if r.params.penalised else () for r in rows],
                [r.seed for r in rows], [len(r.output) for r in rows], want_lp)
            sampled = tokens.tolist()          # the step's one wait for the device
            if logprobs is not None:
                logprobs = logprobs.tolist()
        else:
            torch.cuda.current_stream().synchronize()
        dt = time.perf_counter() - t0
        before = {id(r): len(r.output) for r in rows}
        touched = self.scheduler.commit(plan, sampled, self.model.plan.eos_token_ids)
        for i, r in enumerate(touched):
            new = r.output[before[id(r)]:]
            if logprobs is not None and new:
                r.logprob_sum += logprobs[i]
            outputs.append(self._output(r, new))
        decode = sum(1 for e in plan.entries if e.count == 1 and e.start > 0)
        prefill = plan.num_tokens - decode
        self.stats.steps += 1
        self.stats.decode_tokens += decode
        self.stats.prefill_tokens += prefill
        if prefill:
            self.stats.prefill_seconds += dt
        else:
            self.stats.decode_seconds += dt
        return outputs

    def _output(self, r: Request, new: list[int]) -> GenerationOutput:
        if r.finished:
            self._requests.pop(r.request_id, None)
        return GenerationOutput(self._seq_ids.get(r.request_id, -1), r.request_id, list(new), "", r.finished,
                                r.finish_reason, len(r.prompt), len(r.output), r.logprob_sum)

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
