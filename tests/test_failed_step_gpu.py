"""A step that fails does not stop the engine: its requests end with "error", their pages go back without
becoming known to later requests, and the others are served (the reference's own test of the same property:
tests/test_reprise_apres_exception_8fx.py, for acvram/engine/runner.py:1329-1338).

The failures are made on the host (a step function that raises once; a non-zero code written into the kernels'
status word) or by a wait that is told to give up early (tests/test_kernels_gpu.py); nothing here faults a GPU."""

from __future__ import annotations

import pytest
import torch

import plain_qwen3
from conftest import random_ids
from test_generate_gpu import engine_for

pytestmark = pytest.mark.gpu


def greedy(n):
    from acvram_b200 import SamplingParams
    return SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)


def drain(eng, limit=400):
    outs = []
    for _ in range(limit):
        if eng.idle:
            break
        outs += eng.step()
    assert eng.idle
    return outs


def raise_once_when(eng, request_id, monkeypatch):
    """The runner's step raises the first time a step holds ``request_id`` in its second portion or later."""
    real = eng.runner.step
    state = {"raised": 0}

    def step(entries, device_tokens=None):
        if not state["raised"] and any(e.request == request_id for e in entries) and \
                eng.runner.manager.lengths.get(request_id, 0) > 0:
            state["raised"] += 1
            raise torch.OutOfMemoryError("out of memory, made up by the test")
        return real(entries, device_tokens=device_tokens)

    monkeypatch.setattr(eng.runner, "step", step)
    return state


def test_a_step_that_raises_ends_its_request_and_the_next_one_is_served(tiny_folders, plain_models, monkeypatch):
    cfg, t = plain_models["A"]
    eng = engine_for(tiny_folders["A"], max_batch_size=1, token_budget=16, enable_prefix_cache=True)
    m = eng.runner.manager
    prompt_a, prompt_b = random_ids(cfg["vocab_size"], 40, 1), random_ids(cfg["vocab_size"], 21, 2)
    state = raise_once_when(eng, "a", monkeypatch)
    eng.add_request(prompt_a, greedy(4), "a")
    eng.add_request(prompt_b, greedy(6), "b")
    outs = drain(eng)
    assert state["raised"] == 1
    by = {}
    for o in outs:
        by.setdefault(o.request_id, []).append(o)
    assert by["a"][-1].finished and by["a"][-1].finish_reason == "error" and "out of memory" in by["a"][-1].error
    assert [x for o in by["b"] for x in o.token_ids] == plain_qwen3.greedy_generate(cfg, t, prompt_b, 6)
    assert eng.stats.failed_steps == 1 and eng.stats.failed_requests == 1 and eng.scheduler.counters["failed"] == 1
    # the books balance, and of a's pages only the one that its good first step filled is known
    m.check()
    assert m.free_pages() == [64] and not m.live()
    keys = m.page_keys(prompt_a)
    pool = m.paged_groups[0].pool
    assert pool.lookup(keys[0]) is not None
    assert pool.lookup(keys[1]) is None


def test_requests_of_the_failed_step_end_and_a_waiting_one_is_untouched(tiny_folders, plain_models, monkeypatch):
    cfg, t = plain_models["B"]
    eng = engine_for(tiny_folders["B"], max_batch_size=2, token_budget=24, page_size=8, enable_prefix_cache=True)
    prompts = {k: random_ids(cfg["vocab_size"], n, 10 + n) for k, n in (("a", 30), ("b", 11), ("c", 17))}
    state = raise_once_when(eng, "a", monkeypatch)
    for k, p in prompts.items():
        eng.add_request(p, greedy(5), k)
    outs = drain(eng)
    assert state["raised"] == 1
    last = {o.request_id: o for o in outs if o.finished}
    assert last["a"].finish_reason == "error" and last["b"].finish_reason == "error"
    assert last["c"].finish_reason == "length"
    assert [x for o in outs if o.request_id == "c" for x in o.token_ids] == plain_qwen3.greedy_generate(cfg, t, prompts["c"], 5)
    eng.runner.manager.check()
    assert eng.runner.manager.free_pages() == [64]


@pytest.mark.parametrize("ahead", [False, True])
def test_a_status_code_ends_the_steps_in_flight(tiny_folders, plain_models, ahead):
    """The kernels' status word is read with every step's tokens.  A code in it (here written by the test, as a
    wait that ran out would) fails the step and, when the engine runs one step ahead, the step launched behind it."""
    from acvram_b200.kernels import ops
    cfg, t = plain_models["D"]
    eng = engine_for(tiny_folders["D"], "bfloat16", run_ahead=ahead, max_batch_size=2)
    prompts = [random_ids(cfg["vocab_size"], n, 30 + n) for n in (9, 20)]
    for i, p in enumerate(prompts):
        eng.add_request(p, greedy(40), f"r{i}")
    for _ in range(6):
        eng.step()
    ops.status_word(eng.model.rt.device).fill_(3)
    outs = []
    for _ in range(3):
        outs += eng.step()
    failed = [o for o in outs if o.finish_reason == "error"]
    assert sorted(o.request_id for o in failed) == ["r0", "r1"] and "status 3" in failed[0].error
    assert eng.idle and ops.gemm_status() == 0
    eng.runner.manager.check()
    assert eng.runner.manager.free_pages() == [64]
    # and the engine goes on: a new request gets the plain implementation's tokens (bfloat16: the first few)
    p = random_ids(cfg["vocab_size"], 12, 77)
    got = eng.generate_batch([p], greedy(3))[0]
    ref_logits = plain_qwen3.forward_logits(cfg, t, p)
    assert got[0] == int(ref_logits[-1].argmax())


def test_an_exception_outside_a_step_is_not_swallowed(tiny_folders, monkeypatch):
    """Only what happens between a step's launch and its commit is the engine's to absorb; a fault in the code that
    makes the outputs afterwards (here put there by the test) reaches the caller."""
    eng = engine_for(tiny_folders["A"])
    eng.add_request([1, 2, 3], greedy(2), "a")

    def broken(*a, **k):
        raise KeyError("made up by the test")

    monkeypatch.setattr(eng, "_output", broken)
    with pytest.raises(KeyError):
        for _ in range(5):
            eng.step()
