"""The sampling kernels against the plain sampler."""

from __future__ import annotations

import pytest
import torch

import plain_qwen3

pytestmark = pytest.mark.gpu


def run_sample(logits, temperature, top_k, top_p, min_p, seeds, counters, logprobs=False):
    from acvram_b200.kernels import ops
    R = logits.shape[0]
    dev = "cuda"
    f = lambda v: torch.tensor(v, dtype=torch.float32, device=dev)
    out = torch.empty(R, dtype=torch.int32, device=dev)
    lp = torch.empty(R, dtype=torch.float32, device=dev) if logprobs else None
    ops.sample(logits, f(temperature), torch.tensor(top_k, dtype=torch.int32, device=dev), f(top_p), f(min_p),
               torch.tensor(seeds, dtype=torch.int64, device=dev), torch.tensor(counters, dtype=torch.int64, device=dev),
               out, lp)
    return out.tolist(), (lp.tolist() if logprobs else None)


@pytest.mark.parametrize("V", [331, 4097, 151936])
def test_sample_matches_plain(V):
    g = torch.Generator().manual_seed(V)
    cases = [(0.7, 0, 1.0, 0.0), (1.0, 40, 1.0, 0.0), (1.3, 0, 0.8, 0.0), (0.5, 0, 1.0, 0.05), (0.9, 100, 0.9, 0.01),
             (1.0, 1, 1.0, 0.0), (1.0, 0, 1e-6, 0.0), (0.0, 5, 0.5, 0.1)]
    R = len(cases)
    logits = (torch.randn(R, V, generator=g) * 2.5).cuda()
    seeds = [11 * i + 3 for i in range(R)]
    for counter in (0, 1, 17):
        got, lps = run_sample(logits, [c[0] for c in cases], [c[1] for c in cases], [c[2] for c in cases],
                              [c[3] for c in cases], seeds, [counter] * R, logprobs=True)
        for i, (temp, k, p, mp) in enumerate(cases):
            row = logits[i].cpu()
            if temp <= 0:
                assert got[i] == int(row.argmax())
                continue
            scaled = plain_qwen3.filtered_distribution(row, temp, k, mp, p)
            want = plain_qwen3.draw(scaled, plain_qwen3.philox_uniform(seeds[i], counter))
            assert got[i] == want, f"case {i} counter {counter}"
            assert torch.isfinite(scaled[got[i]]), "a dropped token was drawn"
            assert abs(lps[i] - float(torch.log_softmax(scaled, -1)[got[i]])) < 1e-3


def test_draws_follow_the_distribution():
    """Many counters on one row: the empirical frequencies approach the kept probabilities."""
    V = 50
    g = torch.Generator().manual_seed(1)
    row = torch.randn(V, generator=g) * 2
    n = 4000
    logits = row.repeat(n, 1).cuda()
    got, _ = run_sample(logits, [0.8] * n, [10] * n, [1.0] * n, [0.0] * n, [5] * n, list(range(n)))
    probs = torch.softmax(plain_qwen3.filtered_distribution(row, 0.8, 10, 0.0, 1.0), -1)
    freq = torch.bincount(torch.tensor(got), minlength=V).float() / n
    assert (freq[probs == 0] == 0).all()
    assert (freq - probs).abs().max() < 0.03


def test_penalties():
    from acvram_b200.kernels import ops
    V = 64
    g = torch.Generator().manual_seed(2)
    logits = torch.randn(2, V, generator=g)
    hist = [[3, 3, 9, 11, 3], [5]]
    want = torch.stack([plain_qwen3.penalised(logits[0], hist[0], 1.3, 0.5, 0.2),
                        plain_qwen3.penalised(logits[1], hist[1], 1.0, 0.0, 0.7)])
    dev = logits.cuda()
    rows = torch.tensor([0, 0, 0, 1], dtype=torch.int32).cuda()
    toks = torch.tensor([3, 9, 11, 5], dtype=torch.int32).cuda()
    cnts = torch.tensor([3, 1, 1, 1], dtype=torch.int32).cuda()
    f = lambda v: torch.tensor(v, dtype=torch.float32).cuda()
    ops.apply_penalties(dev, rows, toks, cnts, f([1.3, 1.0]), f([0.5, 0.0]), f([0.2, 0.7]))
    torch.testing.assert_close(dev.cpu(), want, rtol=1e-6, atol=1e-6)


def test_sampler_object_mixes_greedy_and_sampled_rows():
    from acvram_b200.sampling import Sampler, SamplingParams
    V = 300
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(3, V, generator=g) * 2).cuda()
    params = [SamplingParams(temperature=0.0), SamplingParams(temperature=0.8, top_k=20, seed=4),
              SamplingParams(temperature=0.0, repetition_penalty=50.0)]
    best = int(logits[2].argmax())
    toks, _ = Sampler("cuda")(logits, params, [(), (), [best]], [1, 4, 2], [0, 6, 0])
    toks = toks.tolist()
    assert toks[0] == int(logits[0].argmax())
    scaled = plain_qwen3.filtered_distribution(logits[1].cpu(), 0.8, 20, 0.0, 1.0)
    assert toks[1] == plain_qwen3.draw(scaled, plain_qwen3.philox_uniform(4, 6))
    assert toks[2] != best, "the repetition penalty moved the greedy choice"


@pytest.mark.parametrize("V,k", [(331, 5), (4097, 1), (151936, 20), (7, 7), (5, 8)])
def test_top_logprobs_kernel(V, k):
    """The k most probable tokens of each row with logit - logsumexp, against a sort in float64; equal logits
    come lowest id first; a row shorter than k ends with id -1 and -inf."""
    from acvram_b200.kernels import ops
    g = torch.Generator().manual_seed(V + k)
    logits = (torch.randn(6, V, generator=g) * 3.0)
    logits[1, : min(V, 4)] = 2.5                    # equal values among the largest
    logits[2, V // 2] = float("-inf")
    if V > 100:
        logits[3] = torch.round(logits[3])          # many equal values
    ids, lp = ops.top_logprobs(logits.cuda(), k)
    ids, lp = ids.cpu(), lp.cpu()
    ref = torch.log_softmax(logits.double(), dim=-1)
    for r in range(6):
        order = sorted(range(V), key=lambda i: (-float(logits[r, i]), i))
        order = [i for i in order if logits[r, i] != float("-inf")][:k]
        assert ids[r, :len(order)].tolist() == order
        torch.testing.assert_close(lp[r, :len(order)].double(), ref[r, order], rtol=1e-5, atol=1e-5)
        assert all(int(i) == -1 for i in ids[r, len(order):]) and all(v == float("-inf") for v in lp[r, len(order):])
