"""Random weights made on the device are the ones made on the host, bit for bit."""

from __future__ import annotations

import pytest
import torch

from conftest import random_ids, tiny_config

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("role,shape", [("matrix", (301, 77)), ("norm", (130,)), ("embedding", (1000, 96)), ("table", (45, 3)),
                                        ("matrix", (4096, 1030))])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_device_and_host_draw_the_same_values(role, shape, dtype):
    from acvram_b200.weights import TensorNeed, random_tensor
    need = TensorNeed(shape, role)
    host = random_tensor("model.layers.3.some.weight", need, 11, "cpu", dtype)
    dev = random_tensor("model.layers.3.some.weight", need, 11, "cuda:0", dtype)
    assert dev.is_cuda and dev.dtype == host.dtype and dev.shape == host.shape
    assert torch.equal(dev.cpu(), host)


def test_engine_with_random_weights_is_the_folder_of_the_same_seed(tmp_path):
    """``Engine(config, random_weights=True, seed=S)`` and a folder written by ``random-model --seed S`` hold the
    same model: the same tokens, greedy and sampled, in both precisions."""
    from acvram_b200 import Engine, SamplingParams
    from acvram_b200.weights import write_random_model
    cfg = tiny_config("D")
    write_random_model(cfg, tmp_path, seed=9)
    prompts = [random_ids(cfg.vocab_size, n, 60 + n) for n in (7, 40)]
    params = [SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True),
              SamplingParams(temperature=0.8, top_p=0.9, max_tokens=12, ignore_eos=True, seed=5)]
    for dtype in ("float32", "bfloat16"):
        kw = dict(max_batch_size=2, max_model_len=128, page_size=16, num_pages=16)
        from_folder = Engine(str(tmp_path), dtype, **kw).generate_batch(prompts, params)
        from_seed = Engine(cfg, dtype, random_weights=True, seed=9, **kw).generate_batch(prompts, params)
        assert from_folder == from_seed
        other = Engine(cfg, dtype, random_weights=True, seed=10, **kw).generate_batch(prompts, params)
        assert other != from_seed
