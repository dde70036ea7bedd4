"""The plain implementation against the reference's own model code (tests/golden) and against itself."""

from __future__ import annotations

import os

import numpy as np
import torch

import plain_qwen3
from conftest import TINY_SEEDS

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_plain_matches_reference_model_code(plain_models):
    """tests/golden/tiny_*.npz hold logits of the reference's ACVRamModel on the CPU (make_golden.py)."""
    for name in ("A", "B"):
        gold = np.load(os.path.join(GOLDEN, f"tiny_{name}.npz"))
        cfg, t = plain_models[name]
        checksum = float(sum(x.double().abs().sum() for x in t.values()))
        assert abs(checksum - float(gold["weights_abs_sum"])) < 1e-6 * checksum, "random weights changed"
        mine = plain_qwen3.forward_logits(cfg, t, gold["ids"].tolist()).numpy()
        assert np.abs(mine - gold["logits"]).max() < 2e-6
        assert (mine.argmax(-1) == gold["logits"].argmax(-1)).all()


def test_prefix_logits_do_not_depend_on_what_follows(plain_models):
    cfg, t = plain_models["A"]
    ids = list(range(3, 40))
    full = plain_qwen3.forward_logits(cfg, t, ids)
    part = plain_qwen3.forward_logits(cfg, t, ids[:20])
    assert torch.allclose(full[:20], part, atol=1e-6)


def test_qk_norm_comes_before_rotation_and_matters(plain_models):
    """Removing the q/k norms, or swapping norm and rotation, moves the logits (the reference tests the same,
    tests/test_qknorm.py:24-79)."""
    cfg, t = plain_models["B"]
    ids = list(range(5, 30))
    base = plain_qwen3.forward_logits(cfg, t, ids)
    t2 = dict(t)
    for k in t:
        if k.endswith("q_norm.weight") or k.endswith("k_norm.weight"):
            t2[k] = torch.ones_like(t[k])
    assert (plain_qwen3.forward_logits(cfg, t2, ids) - base).abs().max() > 1e-3


def test_window_changes_only_far_queries(plain_models):
    cfg, t = plain_models["A"]
    ids = list(range(7, 47))
    full = plain_qwen3.forward_logits(cfg, t, ids)
    win = plain_qwen3.forward_logits(cfg, t, ids, window=16)
    assert torch.allclose(full[:16], win[:16], atol=1e-6)
    assert (full[30:] - win[30:]).abs().max() > 1e-5


def test_bf16_run_is_near_float32(plain_models):
    cfg, t = plain_models["A"]
    ids = list(range(1, 34))
    a = plain_qwen3.forward_logits(cfg, t, ids)
    b = plain_qwen3.forward_logits(cfg, t, ids, torch.bfloat16)
    d = (a - b).abs().max()
    assert 0 < d < 0.05 * a.abs().max()


def test_philox_known_answers():
    """Philox-4x32-10 known-answer vectors (Random123's kat_vectors): counter and key all zero, and all ones."""
    def words(ctr, key):
        M0, M1, W0, W1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
        c, k = list(ctr), list(key)
        for _ in range(10):
            p0, p1 = M0 * c[0], M1 * c[2]
            c = [((p1 >> 32) ^ c[1] ^ k[0]) & mask, p1 & mask, ((p0 >> 32) ^ c[3] ^ k[1]) & mask, p0 & mask]
            k = [(k[0] + W0) & mask, (k[1] + W1) & mask]
        return c
    assert words([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert words([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    u = plain_qwen3.philox_uniform(0, 0)
    assert abs(u - (0x6627e8d5 + 0.5) / 2 ** 32) < 1e-12


def test_filters_keep_what_the_reference_keeps():
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(200, generator=g) * 3
    s = plain_qwen3.filtered_distribution(logits, 0.7, 10, 0.0, 1.0)
    assert int(torch.isfinite(s).sum()) == 10
    s = plain_qwen3.filtered_distribution(logits, 1.0, 0, 0.0, 0.5)
    p = torch.softmax(logits, -1)
    kept = torch.isfinite(s)
    order = torch.argsort(p, descending=True)
    n = int(kept.sum())
    assert set(order[:n].tolist()) == set(torch.nonzero(kept).flatten().tolist())
    assert p[order[:n - 1]].sum() <= 0.5 < p[order[:n]].sum() + 1e-6
    s = plain_qwen3.filtered_distribution(logits, 1.0, 0, 0.0, 1e-9)
    assert int(torch.isfinite(s).sum()) == 1, "top-p never empties the set"
