"""Shared fixtures: two tiny Qwen3 configurations that differ in every size and option."""

from __future__ import annotations

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with -m gpu)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def tiny_config(which: str):
    """A: 2 layers, hidden 64, 4/2 heads of 16, tied head, eps 1e-6, theta 1e4.
    B: 3 layers, hidden 96, 6/2 heads of 32 (q width 192 != hidden), intermediate 224 and
    vocabulary 384 that are no powers of two, untied head, eps 1e-5, theta 1e6."""
    from acvram_b200.config import Qwen3Config
    if which == "A":
        return Qwen3Config(vocab_size=256, hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
                           rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=True)
    if which == "B":
        return Qwen3Config(vocab_size=384, hidden_size=96, intermediate_size=224, num_hidden_layers=3,
                           num_attention_heads=6, num_key_value_heads=2, head_dim=32, rms_norm_eps=1e-5,
                           rope_theta=1000000.0, max_position_embeddings=512, tie_word_embeddings=False)
    if which == "C":  # odd sizes: 5 q heads on 1 kv head, head 48, hidden 80, vocabulary 331
        return Qwen3Config(vocab_size=331, hidden_size=80, intermediate_size=176, num_hidden_layers=2,
                           num_attention_heads=5, num_key_value_heads=1, head_dim=48, rms_norm_eps=1e-6,
                           rope_theta=50000.0, max_position_embeddings=1024, tie_word_embeddings=False)
    if which == "D":  # head size 64: the bfloat16 runs of this one go through the tensor-core attention kernels
        return Qwen3Config(vocab_size=300, hidden_size=128, intermediate_size=160, num_hidden_layers=2,
                           num_attention_heads=6, num_key_value_heads=2, head_dim=64, rms_norm_eps=1e-6,
                           rope_theta=1000000.0, max_position_embeddings=512, tie_word_embeddings=False)
    if which == "E":  # a width whose rows are not 16-byte aligned (100 elements): the paths beside the tensor-core product
        return Qwen3Config(vocab_size=211, hidden_size=100, intermediate_size=150, num_hidden_layers=2,
                           num_attention_heads=3, num_key_value_heads=3, head_dim=16, rms_norm_eps=1e-6,
                           rope_theta=10000.0, max_position_embeddings=256, tie_word_embeddings=True)
    if which == "F":  # heads of 128, the main head size of the tensor-core kernels; pairs of query heads on a kv head
        return Qwen3Config(vocab_size=512, hidden_size=256, intermediate_size=384, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=128, rms_norm_eps=1e-6,
                           rope_theta=1000000.0, max_position_embeddings=1024, tie_word_embeddings=False)
    if which == "R":  # two layers of the real sizes of Qwen3-8B (the vocabulary alone is small): what serving tiles and splits
        return Qwen3Config(vocab_size=2048, hidden_size=4096, intermediate_size=12288, num_hidden_layers=2,
                           num_attention_heads=32, num_key_value_heads=8, head_dim=128, rms_norm_eps=1e-6,
                           rope_theta=1000000.0, max_position_embeddings=2048, tie_word_embeddings=False)
    raise KeyError(which)


TINY_SEEDS = {"A": 0, "B": 1, "C": 2, "D": 3, "E": 4, "F": 5, "R": 6}
TINY_PAGE = {"A": 16, "B": 8, "C": 16, "D": 16, "E": 16, "F": 64, "R": 64}


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """{name: folder} of the tiny models, written once per session into a temporary folder."""
    from acvram_b200.weights import write_random_model
    out = {}
    for name in ("A", "B", "C", "D", "E", "F"):
        folder = tmp_path_factory.mktemp(f"tiny_{name}")
        write_random_model(tiny_config(name), folder, TINY_SEEDS[name])
        out[name] = str(folder)
    return out


@pytest.fixture(scope="session")
def plain_models(tiny_folders):
    """{name: (config dict, float32 tensors)} as the plain implementation reads them."""
    import plain_qwen3
    return {name: plain_qwen3.read_folder(folder) for name, folder in tiny_folders.items()}


def random_ids(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
