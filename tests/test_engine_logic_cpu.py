"""The step function, the batch builder and the cache on the CPU, with each kernel replaced by its
plain PyTorch reference (tests/kernel_refs.py): only the logic is under test here; the kernels
themselves are tested on the GPU."""

from __future__ import annotations

import dataclasses

import pytest
import torch

import kernel_refs
import plain_qwen3
from acvram_b200.engine.batch import StepEntry
from acvram_b200.engine.runner import ModelRunner
from acvram_b200.models import DecoderModel, plan_of_folder
from acvram_b200.parts import Runtime, ScheduleEntry
from acvram_b200.weights import load_tensors
from conftest import TINY_PAGE, random_ids


@pytest.fixture(autouse=True)
def references_in_place_of_kernels(monkeypatch):
    kernel_refs.patch_ops(monkeypatch)


def build(folder, change_plan=None):
    _, plan = plan_of_folder(folder)
    if change_plan:
        plan = change_plan(plan)
    model = DecoderModel(plan)
    model.load(load_tensors(folder, model.tensor_needs()), Runtime(torch.device("cpu"), torch.float32))
    return model


@pytest.mark.parametrize("name", ["A", "B"])
def test_portions_and_mixing_equal_whole(name, tiny_folders, plain_models):
    cfg, t = plain_models[name]
    model = build(tiny_folders[name])
    ids_a = random_ids(cfg["vocab_size"], 45, 1)
    ids_b = random_ids(cfg["vocab_size"], 23, 2)
    ref_a = plain_qwen3.forward_logits(cfg, t, ids_a)
    ref_b = plain_qwen3.forward_logits(cfg, t, ids_b)
    r = ModelRunner(model, TINY_PAGE[name], 10, 4)
    got_a, got_b = [], []
    got_a.append(r.step([StepEntry("a", ids_a[:19], range(19))]))
    lg = r.step([StepEntry("a", ids_a[19:21], range(2)), StepEntry("b", ids_b[:20], range(20))])
    got_a.append(lg[:2]); got_b.append(lg[2:])
    pa, pb = 21, 20
    while pa < 45 or pb < 23:
        entries = []
        if pb < 23:
            entries.append(StepEntry("b", ids_b[pb:pb + 1], [0]))
        if pa < 45:
            n = min(5, 45 - pa)
            entries.append(StepEntry("a", ids_a[pa:pa + n], range(n)))
        lg = r.step(entries)
        if pb < 23:
            got_b.append(lg[:1]); lg = lg[1:]; pb += 1
        if pa < 45:
            got_a.append(lg); pa += n
    assert (torch.cat(got_a) - ref_a).abs().max() < 2e-6
    assert (torch.cat(got_b) - ref_b).abs().max() < 2e-6
    r.release("a"); r.release("b")
    r.manager.check()
    assert r.manager.free_pages() == [10]


def test_wanted_rows_only(tiny_folders, plain_models):
    cfg, t = plain_models["A"]
    model = build(tiny_folders["A"])
    ids = random_ids(cfg["vocab_size"], 12, 3)
    ref = plain_qwen3.forward_logits(cfg, t, ids)
    r = ModelRunner(model, 16, 4, 2)
    assert r.step([StepEntry("a", ids[:5], ())]).shape == (0, cfg["vocab_size"])
    lg = r.step([StepEntry("a", ids[5:], (6, 0))])
    assert (lg[0] - ref[11]).abs().max() < 2e-6 and (lg[1] - ref[5]).abs().max() < 2e-6


def test_a_layer_twice_and_a_shared_cache(tiny_folders, plain_models):
    """The order of layers is data: layer 1 runs twice (each run with a cache slot of its own)."""
    cfg, t = plain_models["B"]
    sched = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(1, 2), ScheduleEntry(2, 3))
    model = build(tiny_folders["B"], lambda p: dataclasses.replace(p, schedule=sched))
    ids = random_ids(cfg["vocab_size"], 30, 4)
    ref = plain_qwen3.forward_logits(cfg, t, ids, schedule=[0, 1, 1, 2])
    r = ModelRunner(model, 8, 8, 2)
    got = torch.cat([r.step([StepEntry("a", ids[:17], range(17))]), r.step([StepEntry("a", ids[17:], range(13))])])
    assert (got - ref).abs().max() < 2e-6
    assert model.cache_plan().slots_per_group == [4]


def test_reading_another_layers_cache(tiny_folders, plain_models):
    """Layer 2 reads the keys and values that layer 1 wrote (it appends nothing of its own)."""
    cfg, t = plain_models["B"]
    sched = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 1, writes=False))
    model = build(tiny_folders["B"], lambda p: dataclasses.replace(p, schedule=sched))
    assert model.cache_plan().slots_per_group == [2]
    ids = random_ids(cfg["vocab_size"], 21, 5)
    r = ModelRunner(model, 8, 8, 2)
    whole = r.step([StepEntry("w", ids, range(21))])
    r.release("w")
    parts = torch.cat([r.step([StepEntry("p", ids[:9], range(9))]), r.step([StepEntry("p", ids[9:], range(12))])])
    assert (whole - parts).abs().max() < 2e-6, "portions equal whole for a layer that shares a cache"
    base = plain_qwen3.forward_logits(cfg, t, ids)
    assert (whole - base).abs().max() > 1e-4, "and sharing the cache does change the model"


def test_window_layers_get_their_own_group_and_free_pages(tiny_folders, plain_models):
    """A window on some layers: another cache group, pages returned as the window passes."""
    cfg, t = plain_models["A"]

    def windowed(plan):
        layers = list(plan.layers)
        layers[1] = dataclasses.replace(layers[1], mixer=layers[1].mixer.with_params(window=16))
        return dataclasses.replace(plan, layers=tuple(layers))

    model = build(tiny_folders["A"], windowed)
    assert len(model.cache_plan().groups) == 2
    ids = random_ids(cfg["vocab_size"], 80, 6)
    r = ModelRunner(model, 8, 12, 2)
    got = []
    pos = 0
    for n in (30, 2, 17, 1, 1, 1, 28):
        got.append(r.step([StepEntry("a", ids[pos:pos + n], range(n))]))
        pos += n
    got = torch.cat(got)
    full_pages, window_pages = r.manager.free_pages()
    assert full_pages == 12 - 10 and window_pages == 12 - 2, "the windowed group holds only the window's pages"
    # plain: layer 0 full, layer 1 windowed
    s = plain_qwen3.sizes(cfg)
    x = plain_qwen3.embed(t["model.embed_tokens.weight"], torch.tensor(ids), torch.float32)
    positions = torch.arange(80)
    x = plain_qwen3.decoder_layer(x, t, 0, s, positions, 0)
    x = plain_qwen3.decoder_layer(x, t, 1, s, positions, 16)
    ref = plain_qwen3.output_logits(x, t, s)
    assert (got - ref).abs().max() < 2e-6


def test_bad_inputs_are_refused(tiny_folders):
    model = build(tiny_folders["A"])
    r = ModelRunner(model, 16, 4, 2)
    with pytest.raises(ValueError):
        r.step([StepEntry("a", [1, 2, 999], ())])
    with pytest.raises(ValueError):
        r.step([StepEntry("b", [1, 2], (5,))])
    with pytest.raises(ValueError):
        r.step([StepEntry("c", [], ())])


def test_requests_that_take_pages_over_get_the_plain_logits(tiny_folders, plain_models):
    """Scheduler and step function together, with prefix reuse and a pool small enough to preempt: requests whose
    prompts begin alike run behind the pages of earlier ones, and the logits that choose each of their tokens are
    the plain implementation's for the tokens they hold (greedy, so the tokens are the plain ones too)."""
    from acvram_b200.engine.scheduler import Request, Scheduler
    from acvram_b200.sampling import SamplingParams
    cfg, t = plain_models["A"]
    model = build(tiny_folders["A"])
    page = 8
    r = ModelRunner(model, page, 14, 3, enable_prefix_cache=True)
    s = Scheduler(r.manager, 3, 24, 128)
    stem = random_ids(cfg["vocab_size"], 40, 31)
    prompts = [stem[:33], stem[:40], stem[:21] + random_ids(cfg["vocab_size"], 9, 32), stem[:33], stem[:9]]
    reqs = [Request(f"r{i}", list(p), SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True)) for i, p in enumerate(prompts)]
    pending = list(reqs)
    step = 0
    while pending or not s.idle:
        if pending and step % 3 == 0:
            s.add(pending.pop(0))
        plan = s.schedule()
        if plan.entries:
            entries = [StepEntry(e.request.request_id, e.request.token_slice(e.start, e.count),
                                 (e.count - 1,) if e.samples else ()) for e in plan.entries]
            logits = r.step(entries)
            rows = [e.request for e in plan.entries if e.samples]
            for req, row in zip(rows, logits):
                want = plain_qwen3.forward_logits(cfg, t, req.tokens)[-1]
                assert (row - want).abs().max() < 5e-6, f"{req.request_id} at {len(req.tokens)} tokens (took over {req.reused})"
            s.commit(plan, [int(row.argmax()) for row in logits])
        r.manager.check()
        step += 1
        assert step < 400
    for req, p in zip(reqs, prompts):
        assert req.output == plain_qwen3.greedy_generate(cfg, t, p, 7)
    assert s.counters["reused_tokens"] >= 32 + 16 + 32 and r.manager.free_pages() == [14]


def test_step_cost_follows_the_plan(tiny_folders, plain_models):
    """What a step reads and computes, as the parts report it, against the sums written out for this architecture."""
    cfg, _ = plain_models["B"]
    model = build(tiny_folders["B"])
    L, H, I, V = cfg["num_hidden_layers"], cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    NH, NKV, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    matrices = L * (H * (NH + 2 * NKV) * D + NH * D * H + 3 * H * I) + V * H
    norms = L * (2 * H + 2 * D) + H
    q_lens, kv_lens = [1, 1, 5], [30, 7, 12]
    cost = model.step_cost(q_lens, kv_lens, logit_rows=3)
    assert cost["weight_bytes"] == 4 * (matrices + norms)              # a float32 model; norm weights are float32 too
    assert cost["cache_bytes"] == L * 2 * sum(kv_lens) * NKV * D * 4
    seen = 30 + 7 + sum(range(8, 13))                                   # keys that each query sees
    want = 2.0 * 7 * (matrices - V * H) + 2.0 * 3 * V * H + L * 4.0 * NH * D * seen
    assert abs(cost["flops"] - want) < 1e-6 * want
    # a layer that runs twice is read twice
    twice = build(tiny_folders["B"], lambda p: dataclasses.replace(
        p, schedule=p.schedule + (ScheduleEntry(0, p.num_cache_slots, True),)))
    assert twice.step_cost([1], [5], 1)["weight_bytes"] > model.step_cost([1], [5], 1)["weight_bytes"]


def test_the_plan_of_a_product_follows_its_shape():
    """Which tile form a tensor-core product takes, for a device of 148 multiprocessors: weights on the tile's rows up to
    128 tokens (split along K where the tiles alone do not fill the device), tokens on the rows above; pairs of CTAs on
    256 x 256 where their rounds cost less than any width of one CTA's tile, whole heads in a tile where the epilogue
    wants them."""
    from acvram_b200.kernels import ops
    plan = lambda *a, **k: ops.gemm_tc_plan(*a, sms=148, **k)
    for M in (1, 8, 16):
        swap, bn, splits, stages = plan(M, 4096, 4096)[:4]
        assert (swap, bn) == (1, 16) and splits > 1, "32 tiles of weights on 148 SMs: the K range is shared out"
    assert plan(100, 6144, 4096)[:2] == (1, 128)
    for shape in ((2048, 6144, 4096), (2048, 4096, 4096), (2048, 24576, 4096), (2048, 4096, 12288), (8192, 24576, 4096)):
        p = plan(*shape)
        assert p[:3] == (0, 256, 1) and p[4] == ops.GEMM_PAIR, shape
    assert len(plan(1056, 34816, 5120)) == 4 and plan(1056, 34816, 5120)[:2] == (0, 256)      # 1280 rows of pair tiles for 1056 tokens
    assert plan(1056, 5120, 5120)[:2] == (0, 160), "a narrower tile where it saves a round"
    assert plan(1056, 5120, 5120, bn_multiple=128)[1] % 128 == 0
    assert plan(300, 200, 512)[:2] == (0, 128) and plan(300, 40, 512)[:2] == (0, 64)
    # a device with one multiprocessor has no pairs
    assert len(ops.gemm_tc_plan(2048, 4096, 4096, sms=1)) == 4


def test_the_splits_of_decode_attention_follow_what_fits_the_device(monkeypatch):
    """How the split-KV kernel cuts the context, for a device that holds 296 of its CTAs at once (stubbed: the real
    figure is asked of the runtime): a few long requests are split so far that a CTA's own streaming is short, many
    requests not at all; more than 8 splits, through scratch memory, only where 8 leave a CTA thousands of keys; and
    where the clusters of some size fit the device badly, that size is passed over."""
    from acvram_b200.kernels import ops
    fits = {}

    def resident(num_heads, num_kv_heads, head_dim, page_size, n_splits, pages_of_split, cluster_merge, alone=False):
        if alone:       # one CTA to an SM, 148 SMs: whole clusters only
            return {1: 148, 2: 148, 4: 132, 6: 132, 8: 120}[n_splits if cluster_merge else 1]
        return fits.get((n_splits, cluster_merge), 296)
    monkeypatch.setattr(ops, "decode_resident", resident)
    plan = lambda n_dec, max_kv: ops.decode_plan.__wrapped__(n_dec, 32, 8, 128, 64, max_kv)
    assert plan(64, 2048) == (1, False) and plan(64, 16384) == (1, False)
    n, in_clusters = plan(8, 2048)
    assert 2 <= n <= 4 and in_clusters
    n, in_clusters = plan(1, 8192)
    assert n == 8 and in_clusters
    n, in_clusters = plan(1, 65536)
    assert n > 8 and not in_clusters
    assert plan(1, 300) == (1, False), "no split shorter than 256 keys"
    # 24 clusters of 8 for 3 requests: all at once on this device, not on one that holds 15 of them
    assert plan(3, 16384) == (8, True)
    fits[(8, True)] = 120
    assert plan(3, 16384)[0] != 8 or not plan(3, 16384)[1]
    # the cost itself: a second round costs, and so does every split's share of the merge
    one = ops.decode_splits_cost(2, 8, 8192, 8, True, 296, 512)
    assert ops.decode_splits_cost(2, 8, 8192, 8, True, 64, 512) > 1.3 * one
    assert ops.decode_splits_cost(2, 8, 8192, 8, False, 296, 512) > one
