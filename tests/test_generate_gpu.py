"""Generation through the Python entry point and the command line, against the plain implementation."""

from __future__ import annotations

import json
import os
import subprocess
import sys

import pytest
import torch

import plain_qwen3
from conftest import ROOT, TINY_PAGE, random_ids

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype="float32", **kw):
    from acvram_b200 import Engine
    args = dict(max_batch_size=4, max_model_len=256, page_size=16, num_pages=64, token_budget=64)
    args.update(kw)
    return Engine(folder, dtype, **args)


def test_greedy_three_requests_tiny_a(tiny_folders, plain_models):
    """Tiny A's workload: prompts of 5/17/33 tokens, 16 greedy tokens each, generated together."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["A"]
    prompts = [random_ids(cfg["vocab_size"], n, 200 + n) for n in (5, 17, 33)]
    eng = engine_for(tiny_folders["A"], page_size=TINY_PAGE["A"])
    got = eng.generate_batch(prompts, SamplingParams(temperature=0.0, max_tokens=16, ignore_eos=True))
    for p, g in zip(prompts, got):
        assert g == plain_qwen3.greedy_generate(cfg, t, p, 16)
    assert eng.runner.manager.free_pages() == [64] and eng.idle
    assert eng.stats.decode_tokens == 3 * 15 and eng.stats.prefill_tokens == 55


def test_generate_iterator_and_stats(tiny_folders, plain_models):
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["B"]
    prompt = random_ids(cfg["vocab_size"], 9, 3)
    eng = engine_for(tiny_folders["B"], page_size=8)
    outs = list(eng.generate(prompt, SamplingParams(temperature=0.0, max_tokens=5, ignore_eos=True)))
    toks = [x for o in outs for x in o.token_ids]
    assert toks == plain_qwen3.greedy_generate(cfg, t, prompt, 5)
    assert outs[-1].finished and outs[-1].finish_reason == "length" and outs[-1].completion_tokens == 5
    assert outs[0].prompt_tokens == 9 and not outs[0].finished


def test_long_greedy_decoding(tiny_folders, plain_models):
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["A"]
    prompt = random_ids(cfg["vocab_size"], 7, 5)
    eng = engine_for(tiny_folders["A"])
    got = eng.generate_batch([prompt], SamplingParams(temperature=0.0, max_tokens=200, ignore_eos=True))[0]
    assert got == plain_qwen3.greedy_generate(cfg, t, prompt, 200)


def test_temperature_sampling_tiny_b_portions_mixed_with_decoding(tiny_folders, plain_models):
    """Tiny B's workload: prompts of 1/9/40/130 tokens in portions of 32 beside decoding, temperature 0.7, fixed
    seeds.  Each sampled token must be the plain sampler's choice on the plain logits with the same uniform."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["B"]
    prompts = [random_ids(cfg["vocab_size"], n, 300 + n) for n in (1, 9, 40, 130)]
    eng = engine_for(tiny_folders["B"], page_size=8, num_pages=128, token_budget=32)
    params = [SamplingParams(temperature=0.7, top_k=50, top_p=0.9, max_tokens=12, seed=1000 + i, ignore_eos=True)
              for i in range(4)]
    got = eng.generate_batch(prompts, params)
    for i, (p, g) in enumerate(zip(prompts, got)):
        assert len(g) == 12
        logits = plain_qwen3.forward_logits(cfg, t, p + g)
        for n, tok in enumerate(g):
            row = logits[len(p) - 1 + n]
            scaled = plain_qwen3.filtered_distribution(row, 0.7, 50, 0.0, 0.9)
            want = plain_qwen3.draw(scaled, plain_qwen3.philox_uniform(1000 + i, n))
            assert tok == want, f"request {i} token {n}: engine {tok}, plain sampler {want}"


def test_a_requests_tokens_do_not_depend_on_the_batch(tiny_folders, plain_models):
    from acvram_b200 import SamplingParams
    cfg, _ = plain_models["B"]
    prompts = [random_ids(cfg["vocab_size"], n, 400 + n) for n in (12, 30, 5)]
    sp = lambda i: SamplingParams(temperature=0.9, top_p=0.95, max_tokens=10, seed=77 + i, ignore_eos=True)
    eng = engine_for(tiny_folders["B"], page_size=8)
    together = eng.generate_batch(prompts, [sp(i) for i in range(3)])
    alone = [eng.generate_batch([p], sp(i))[0] for i, p in enumerate(prompts)]
    assert together == alone


def test_preemption_changes_no_token(tiny_folders, plain_models):
    """With so few pages that running requests are preempted and recomputed, greedy tokens stay the same."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["A"]
    prompts = [random_ids(cfg["vocab_size"], n, 500 + n) for n in (20, 25, 18)]
    sp = SamplingParams(temperature=0.0, max_tokens=30, ignore_eos=True)
    small = engine_for(tiny_folders["A"], num_pages=7, token_budget=16)
    got = small.generate_batch(prompts, sp)
    assert small.stats.preempted > 0, "the pool was meant to be too small"
    for p, g in zip(prompts, got):
        assert g == plain_qwen3.greedy_generate(cfg, t, p, 30)
    small.runner.manager.check()
    assert small.runner.manager.free_pages() == [7]


def test_refusal_and_stop_tokens(tiny_folders, plain_models):
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["A"]
    eng = engine_for(tiny_folders["A"], num_pages=2)
    outs = list(eng.generate(random_ids(cfg["vocab_size"], 40, 1), SamplingParams(temperature=0.0, max_tokens=4)))
    assert outs[-1].finished and outs[-1].finish_reason == "refused" and outs[-1].token_ids == []
    eng = engine_for(tiny_folders["A"])
    prompt = random_ids(cfg["vocab_size"], 10, 2)
    free = plain_qwen3.greedy_generate(cfg, t, prompt, 6)
    outs = list(eng.generate(prompt, SamplingParams(temperature=0.0, max_tokens=6, stop_token_ids=[free[2]])))
    toks = [x for o in outs for x in o.token_ids]
    assert toks == free[:free.index(free[2]) + 1] and outs[-1].finish_reason == "stop"


def test_bfloat16_generation_follows_the_plain_logits(tiny_folders, plain_models):
    """bfloat16 greedy tokens: at every step the engine's choice is within the plain float32 logits' near-ties."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["B"]
    prompt = random_ids(cfg["vocab_size"], 33, 9)
    eng = engine_for(tiny_folders["B"], "bfloat16", page_size=8)
    got = eng.generate_batch([prompt], SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))[0]
    logits = plain_qwen3.forward_logits(cfg, t, prompt + got)
    ref16 = plain_qwen3.forward_logits(cfg, t, prompt + got, torch.bfloat16)
    yard = float((logits - ref16).abs().max())
    for n, tok in enumerate(got):
        row = logits[len(prompt) - 1 + n]
        assert float(row.max() - row[tok]) <= 3 * yard, f"token {n} is not a near-best choice"


def test_command_line_generate_and_random_model(tiny_folders, plain_models, tmp_path):
    cfg, t = plain_models["A"]
    prompt = random_ids(cfg["vocab_size"], 11, 4)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "acvram"), "generate", tiny_folders["A"],
                          "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5",
                          "--temperature", "0", "--ignore-eos", "--max-model-len", "128", "--num-pages", "16",
                          "--json"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["outputs"][0] == plain_qwen3.greedy_generate(cfg, t, prompt, 5)
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "acvram"), "random-model",
                          os.path.join(tiny_folders["B"], "config.json"), str(tmp_path / "m"), "--seed", "1"],
                         capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    from safetensors.torch import load_file
    a = load_file(os.path.join(tiny_folders["B"], "model.safetensors"))
    b = load_file(str(tmp_path / "m" / "model.safetensors"))
    assert all(torch.equal(a[k], b[k]) for k in a)
    # `bench --what decode` (the reference's name): a rate for each batch size asked for
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "acvram"), "bench", tiny_folders["A"], "--what", "decode",
                          "--batch", "1,3", "--context", "20", "--tokens", "8", "--prefill", "40", "--json"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["decode_b1"]["tokens_per_s"] > 0 and res["decode_b3"]["tokens_per_s"] > res["decode_b1"]["tokens_per_s"] * 0.5
    assert res["prefill"]["tokens"] == 40 and res["prefill"]["tokens_per_s"] > 0
    # `bench --what kernels`: the hot kernels one by one, here two cases of them
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "acvram"), "bench", "--what", "kernels", "--case",
                          "gemm_decode,attention_decode", "--json"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    res = json.loads(out.stdout.strip().splitlines()[-1])
    assert res["gemm_decode"]["kernel"] == "gemm_tc" and res["gemm_decode"]["weights_gbs"] > 100
    assert res["attention_decode"]["pages_gbs"] > 100


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_running_one_step_ahead_changes_no_token(tiny_folders, plain_models, dtype):
    """The engine launches a decode step before it has read the tokens of the step before it.  Requests that end on
    a token of their own (a stop token), by their length, at different times, with seeded sampling: the same tokens,
    the same finish reasons, every page back."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["A"]
    prompts = [random_ids(cfg["vocab_size"], n, 300 + n) for n in (4, 19, 33, 8)]
    ref = engine_for(tiny_folders["A"], dtype, run_ahead=False, page_size=TINY_PAGE["A"]).generate_batch(
        prompts, SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True))
    params = [SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True),
              SamplingParams(temperature=0.8, top_p=0.9, seed=11, max_tokens=13, ignore_eos=True),
              SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True, stop_token_ids=[ref[2][6]]),
              SamplingParams(temperature=0.0, max_tokens=1, ignore_eos=True)]
    results = []
    for ahead in (False, True):
        eng = engine_for(tiny_folders["A"], dtype, run_ahead=ahead, page_size=TINY_PAGE["A"])
        ids = [eng.add_request(p, sp) for p, sp in zip(prompts, params)]
        got = {i: ([], None) for i in ids}
        calls = 0
        while not eng.idle:
            calls += 1
            for out in eng.step():
                toks, _ = got[out.request_id]
                got[out.request_id] = (toks + out.token_ids, out.finish_reason if out.finished else None)
        assert eng.runner.manager.free_pages() == [64]
        eng.runner.manager.check()
        results.append([got[i] for i in ids])
    assert results[0] == results[1]
    assert results[1][0] == (ref[0], "length") and results[1][2][1] == "stop" and len(results[1][2][0]) <= 7
    assert len(results[1][1][0]) == 13 and len(results[1][3][0]) == 1


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_traffic_gives_the_same_tokens_one_step_ahead_or_not(tiny_folders, plain_models, dtype):
    """Random requests (greedy, seeded sampling, stop tokens, lengths from 1 token up) arriving at random steps into
    pools small enough to preempt and to make requests wait: every request gets the same tokens and the same end
    whether the engine runs one step ahead or not, and every page comes back."""
    import random
    from acvram_b200 import SamplingParams
    cfg, _ = plain_models["A"]
    vocab = cfg["vocab_size"]

    def run(seed, ahead):
        rng = random.Random(seed)
        pages = rng.choice([10, 14, 40])
        eng = engine_for(tiny_folders["A"], dtype, run_ahead=ahead, page_size=16, num_pages=pages, max_model_len=200,
                         token_budget=rng.choice([8, 32, 64]))
        reqs = []
        for i in range(rng.randint(3, 8)):
            prompt = [rng.randrange(vocab) for _ in range(rng.randint(1, 60))]
            kind = rng.random()
            if kind < 0.5:
                sp = SamplingParams(temperature=0.0, max_tokens=rng.randint(1, 40), ignore_eos=rng.random() < 0.5)
            elif kind < 0.8:
                sp = SamplingParams(temperature=0.9, top_p=0.9, top_k=rng.choice([0, 5]), seed=rng.randrange(1000),
                                    max_tokens=rng.randint(1, 40), ignore_eos=True)
            else:
                sp = SamplingParams(temperature=0.0, max_tokens=rng.randint(5, 40), ignore_eos=True,
                                    stop_token_ids=[rng.randrange(vocab) for _ in range(40)])
            reqs.append((prompt, sp, rng.randint(0, 30)))
        got, step, pending = {}, 0, list(enumerate(reqs))
        while pending or not eng.idle:
            for k, (p, sp, at) in list(pending):
                if at <= step:
                    eng.add_request(p, sp, request_id=f"r{k}")
                    pending.remove((k, (p, sp, at)))
            for o in eng.step():
                toks, _ = got.get(o.request_id, ([], None))
                got[o.request_id] = (toks + o.token_ids, o.finish_reason if o.finished else None)
            step += 1
            assert step < 3000
        eng.runner.manager.check()
        assert eng.runner.manager.free_pages() == [pages]
        return got, eng.stats.preempted

    preempted = 0
    for seed in range(10):
        a, pa = run(seed, False)
        b, pb = run(seed, True)
        assert a == b, f"seed {seed}"
        assert all(reason is not None for _, reason in a.values())
        preempted += pa + pb
    assert preempted > 0       # the small pools did make requests give way


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pages_taken_over_change_no_token(tiny_folders, plain_models, dtype):
    """Prefix reuse: a prompt seen before, prompts that begin like it (one of them cut inside a page), and a
    pool so small that kept pages lose their room on the way.  What a request generates is what it would have
    generated alone: in float32 the plain implementation's tokens, in bfloat16 near-best choices of its logits."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["B"]
    vocab = cfg["vocab_size"]
    base = random_ids(vocab, 50, 77)
    prompts = [base, list(base), base[:40] + random_ids(vocab, 21, 78), base[:33], random_ids(vocab, 30, 79), list(base)]
    sp = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)
    eng = engine_for(tiny_folders["B"], dtype, page_size=8, num_pages=14, max_model_len=128)
    reused, outs = [], []
    for p in prompts:                   # one after the other: each finds what the earlier ones left
        outs.append(eng.generate_batch([p], sp)[0])
        reused.append(eng.stats.reused_tokens - sum(reused))
        eng.runner.manager.check()
    assert reused[0] == 0 and reused[1] == 48 and reused[2] == 40 and reused[3] == 32 and reused[4] == 0
    assert eng.runner.manager.free_pages() == [14] and eng.runner.manager.paged_groups[0].pool.num_kept > 0
    for p, g in zip(prompts, outs):
        if dtype == "float32":
            assert g == plain_qwen3.greedy_generate(cfg, t, p, 10)
        else:
            logits = plain_qwen3.forward_logits(cfg, t, p + g)
            yard = float((logits - plain_qwen3.forward_logits(cfg, t, p + g, torch.bfloat16)).abs().max())
            for n, tok in enumerate(g):
                row = logits[len(p) - 1 + n]
                assert float(row.max() - row[tok]) <= 3 * yard, f"token {n} is not a near-best choice"
    # the same requests all at once, and without reuse: the same tokens in float32
    if dtype == "float32":
        for cache in (True, False):
            eng2 = engine_for(tiny_folders["B"], dtype, page_size=8, num_pages=64, max_model_len=128,
                              enable_prefix_cache=cache)
            assert eng2.generate_batch(prompts, sp) == outs
            assert eng2.stats.reused_tokens == 0 or cache


@pytest.mark.parametrize("ahead", [False, True])
def test_abort_between_steps_frees_everything_and_leaves_the_others_alone(tiny_folders, plain_models, ahead):
    """A request is aborted while it decodes (with the engine one step ahead: while a step that holds its token is
    unread), another while it still waits: their pages come back at once, nothing more is delivered for them, and
    the requests beside them get the tokens they would have got alone."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["A"]
    prompts = [random_ids(cfg["vocab_size"], n, 400 + n) for n in (20, 33, 7, 50, 12)]
    sp = SamplingParams(temperature=0.0, max_tokens=24, ignore_eos=True)
    eng = engine_for(tiny_folders["A"], run_ahead=ahead, max_batch_size=3, num_pages=24)
    ids = [eng.add_request(p, sp, request_id=f"q{i}") for i, p in enumerate(prompts)]
    got = {i: [] for i in ids}
    after_abort = {}
    step = 0
    while not eng.idle:
        if step == 6:
            eng.abort("q1")                     # decoding
            eng.abort("q4")                     # still waiting: three requests are live at most
            after_abort = {k: len(v) for k, v in got.items()}
        for o in eng.step():
            got[o.request_id].extend(o.token_ids)
        step += 1
        assert step < 500
    assert len(got["q1"]) == after_abort["q1"] < 24 and got["q4"] == []
    for i in (0, 2, 3):
        assert got[f"q{i}"] == plain_qwen3.greedy_generate(cfg, t, prompts[i], 24)
    eng.runner.manager.check()
    assert eng.runner.manager.free_pages() == [24]


def test_log_probabilities_of_the_chosen_and_of_the_most_probable_tokens(tiny_folders, plain_models):
    """``logprobs=k``: every delivered token comes with its own log probability and with the k most probable tokens
    of its step, normalised over the whole vocabulary of the plain implementation's logits; a request beside it
    that asked for none gets none."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["B"]
    prompts = [random_ids(cfg["vocab_size"], n, 500 + n) for n in (11, 23)]
    eng = engine_for(tiny_folders["B"], page_size=8)
    a = eng.add_request(prompts[0], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True, logprobs=3))
    b = eng.add_request(prompts[1], SamplingParams(temperature=0.0, max_tokens=6, ignore_eos=True))
    outs = {a: [], b: []}
    while not eng.idle:
        for o in eng.step():
            outs[o.request_id].append(o)
    assert all(o.logprob is None and o.top_logprobs is None and o.cumulative_logprob is None for o in outs[b])
    toks = [x for o in outs[a] for x in o.token_ids]
    assert toks == plain_qwen3.greedy_generate(cfg, t, prompts[0], 6)
    ref = torch.log_softmax(plain_qwen3.forward_logits(cfg, t, prompts[0] + toks).double(), dim=-1)
    total = 0.0
    for n, o in enumerate(outs[a]):
        row = ref[len(prompts[0]) - 1 + n]
        want = torch.topk(row, 3)
        assert [i for i, _ in o.top_logprobs] == want.indices.tolist()
        assert o.top_logprobs[0][0] == o.token_ids[0], "greedy: the chosen token is the most probable one"
        torch.testing.assert_close(torch.tensor([p for _, p in o.top_logprobs]).double(), want.values, rtol=1e-4, atol=1e-4)
        assert abs(o.logprob - float(row[o.token_ids[0]])) < 1e-4
        total += o.logprob
        assert abs(o.cumulative_logprob - total) < 1e-4


@pytest.mark.parametrize("ahead", [False, True])
def test_text_deltas_and_stop_strings_with_a_tokenizer(tiny_folders, plain_models, ahead):
    """With a tokenizer the outputs carry their text, and a stop string ends its request where it begins: the
    string is not delivered, the pages come back, the request beside it is not touched."""
    from acvram_b200 import SamplingParams

    class Tok:
        def decode(self, ids):
            return "".join(f"<{i}>" for i in ids)

    cfg, t = plain_models["A"]
    prompts = [random_ids(cfg["vocab_size"], n, 600 + n) for n in (9, 14)]
    want = [plain_qwen3.greedy_generate(cfg, t, p, 12) for p in prompts]
    j = want[0].index(want[0][5])          # the stop string is the text of the sixth token: it ends the request where it first occurs
    eng = engine_for(tiny_folders["A"], run_ahead=ahead, tokenizer=Tok())
    a = eng.add_request(prompts[0], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True, stop=[f"<{want[0][j]}>"]))
    b = eng.add_request(prompts[1], SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    outs = {a: [], b: []}
    while not eng.idle:
        for o in eng.step():
            outs[o.request_id].append(o)
    assert "".join(o.text_delta for o in outs[b]) == "".join(f"<{i}>" for i in want[1])
    assert outs[b][-1].finish_reason == "length"
    assert "".join(o.text_delta for o in outs[a]) == "".join(f"<{i}>" for i in want[0][:j])
    assert outs[a][-1].finished and outs[a][-1].finish_reason == "stop"
    assert [x for o in outs[a] for x in o.token_ids] == want[0][:j + 1], "the token that completed the string is the last"
    assert eng.runner.manager.free_pages() == [64]
    eng.runner.manager.check()


def test_generation_with_the_layers_as_single_kernels(tiny_folders, plain_models):
    """``Engine(fuse_decode_layers=True)``: decode steps of up to 16 requests run each layer as one persistent kernel;
    the tokens follow the plain implementation's logits as the ordinary path's do."""
    from acvram_b200 import SamplingParams
    cfg, t = plain_models["F"]
    prompts = [random_ids(cfg["vocab_size"], n, 300 + n) for n in (5, 70, 131)]
    sp = SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True)
    fused = engine_for(tiny_folders["F"], "bfloat16", page_size=16, max_model_len=512, fuse_decode_layers=True)
    plain = engine_for(tiny_folders["F"], "bfloat16", page_size=16, max_model_len=512)
    got_f, got_p = fused.generate_batch(prompts, sp), plain.generate_batch(prompts, sp)
    assert fused.stats.failed_steps == 0 and all(b.fuse_decode for b in fused.model.blocks)
    for p, gf, gp in zip(prompts, got_f, got_p):
        ref = plain_qwen3.forward_logits(cfg, t, p)
        assert gf[0] == gp[0] == int(ref[-1].argmax())
    # from then on each path follows its own roundings; both stay close to the plain model's choice at every step
    for p, gf in zip(prompts, got_f):
        ids = list(p)
        for tok in gf:
            lg = plain_qwen3.forward_logits(cfg, t, ids)[-1]
            assert float(lg.max() - lg[tok]) < 0.05, "a token far from the plain model's best"
            ids.append(tok)
