"""The persistent decode-layer kernel (one launch for a whole layer of a small decode step) against the separate
kernels and against the plain implementation."""

from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_qwen3
from conftest import TINY_SEEDS, random_ids, tiny_config

pytestmark = pytest.mark.gpu


def config_g():
    """Heads of 64 (two heads to a tile of 128 features), four kv heads, sizes that are multiples of 64 only."""
    from acvram_b200.config import Qwen3Config
    return Qwen3Config(vocab_size=400, hidden_size=192, intermediate_size=448, num_hidden_layers=3, num_attention_heads=8,
                       num_key_value_heads=4, head_dim=64, rms_norm_eps=1e-5, rope_theta=10000.0,
                       max_position_embeddings=1024, tie_word_embeddings=True)


def build(name, tmp_path_factory):
    from acvram_b200.models import build_from_folder
    from acvram_b200.weights import write_random_model
    cfg = config_g() if name == "G" else tiny_config(name)
    folder = str(tmp_path_factory.mktemp(f"dl_{name}"))
    write_random_model(cfg, folder, TINY_SEEDS.get(name, 7))
    _, model = build_from_folder(folder, torch.bfloat16)
    return cfg, model, plain_qwen3.read_folder(folder)


@pytest.mark.parametrize("name,page,lens,graphs", [("F", 16, [70, 3, 129, 300, 17], False), ("F", 64, [70, 3, 129], True),
                                                   ("G", 16, [33, 200, 64, 65, 1, 500, 90, 12, 7], False),
                                                   ("G", 32, [33, 200], True),
                                                   ("R", 16, [40, 513, 130, 5, 260, 17, 64, 9], True),
                                                   ("R", 16, [700], False)])
def test_fused_layer_equals_the_separate_kernels_and_the_plain_model(name, page, lens, graphs, tmp_path_factory):
    from acvram_b200.engine.batch import StepEntry
    from acvram_b200.engine.runner import ModelRunner
    from acvram_b200.kernels import ops
    cfg, model, (pcfg, pt) = build(name, tmp_path_factory)
    reqs = {f"r{i}": random_ids(cfg.vocab_size, n + 6, 70 + i) for i, n in enumerate(lens)}
    n_dec = 6

    def run(fused: bool):
        for b in model.blocks:
            b.fuse_decode = fused
        runner = ModelRunner(model, page, sum(-(-len(v) // page) for v in reqs.values()) + 4, len(reqs))
        if graphs:
            runner.enable_graphs()
        runner.step([StepEntry(k, v[:-n_dec], ()) for k, v in reqs.items()])
        before = ops.LAUNCHES + runner.graph_launches
        out = []
        for i in range(n_dec, 0, -1):
            lg = runner.step([StepEntry(k, v[len(v) - i:len(v) - i + 1], (0,)) for k, v in reqs.items()])
            out.append(lg.float().cpu().numpy())
        launches = ops.LAUNCHES + runner.graph_launches - before
        runner.check_status()
        return np.stack(out), launches

    sep, launches_sep = run(False)
    fus, launches_fus = run(True)
    n_layers = len(model.blocks)
    assert launches_sep - launches_fus >= n_dec * n_layers * 4, "the fused path did not run"
    ref = {k: plain_qwen3.forward_logits(pcfg, pt, v).numpy() for k, v in reqs.items()}
    ref16 = {k: plain_qwen3.forward_logits(pcfg, pt, v, torch.bfloat16).numpy() for k, v in reqs.items()}
    yard = max(float(np.abs(ref16[k] - ref[k]).max()) for k in ref)
    worst_f = worst_s = 0.0
    for s, i in enumerate(range(n_dec, 0, -1)):
        for row, (k, v) in enumerate(reqs.items()):
            want = ref[k][len(v) - i]
            worst_f = max(worst_f, float(np.abs(fus[s, row] - want).max()))
            worst_s = max(worst_s, float(np.abs(sep[s, row] - want).max()))
    assert worst_s <= 2.5 * yard
    assert worst_f <= 2.5 * yard, f"fused: {worst_f:.3e}, separate: {worst_s:.3e}, bfloat16 yardstick {yard:.3e}"
    assert float(np.abs(fus - sep).max()) <= 2.5 * yard
