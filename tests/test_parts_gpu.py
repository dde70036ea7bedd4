"""Each part alone on the GPU against the plain implementation's function for it."""

from __future__ import annotations

import pytest
import torch

import plain_qwen3
from conftest import random_ids

pytestmark = pytest.mark.gpu


def ctx_for(runner, request, tokens, want=()):
    from acvram_b200.engine.batch import StepEntry
    return runner.prepare([StepEntry(request, tokens, want)])


@pytest.fixture()
def model_and_plain(tiny_folders, plain_models):
    def make(name, dtype=torch.float32):
        from acvram_b200.engine.runner import ModelRunner
        from acvram_b200.models import build_from_folder
        _, model = build_from_folder(tiny_folders[name], dtype, "cuda:0")
        cfg, t = plain_models[name]
        return model, ModelRunner(model, 8, 64, 4), cfg, t, plain_qwen3.sizes(cfg)
    return make


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_norm_part(name, model_and_plain):
    model, _, cfg, t, s = model_and_plain(name)
    x = torch.randn(9, s["H"], device="cuda")
    d = torch.randn(9, s["H"], device="cuda")
    norm = model.blocks[1].post_norm
    want_x = x.cpu() + d.cpu()
    want = plain_qwen3.rms_norm(want_x, t["model.layers.1.post_attention_layernorm.weight"], s["eps"])
    got = norm.forward(x, d)
    torch.testing.assert_close(x.cpu(), want_x, rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_rotary_table(name, model_and_plain):
    model, _, cfg, t, s = model_and_plain(name)
    table = model.blocks[0].mixer.position.rotary_table().cpu()
    pos = torch.tensor([0, 1, 17, cfg["max_position_embeddings"] - 1])
    cos, sin = plain_qwen3.rotary_tables(pos, s["D"], s["theta"])
    half = s["D"] // 2
    torch.testing.assert_close(table[pos, :half], cos[:, :half], rtol=0, atol=0)
    torch.testing.assert_close(table[pos, half:], sin[:, :half], rtol=0, atol=0)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_attention_mixer_in_portions(name, model_and_plain):
    """The mixer alone on a sequence fed as three portions equals the plain attention block on the whole."""
    from acvram_b200.parts import CacheView
    model, runner, cfg, t, s = model_and_plain(name)
    mixer = model.blocks[1].mixer
    n = 41
    h = torch.randn(n, s["H"]) * 0.5
    want = plain_qwen3.attention_block(h, t, "model.layers.1.", s, torch.arange(n))
    k, v = runner.storage.pages(1)
    got = []
    pos = 0
    for m in (17, 2, 22):
        ctx = ctx_for(runner, "a", [1] * m)
        got.append(mixer.forward(h[pos:pos + m].cuda(), ctx, CacheView(0, True, k_pages=k, v_pages=v)))
        runner.manager.advance("a", pos + m)
        pos += m
    torch.testing.assert_close(torch.cat(got).cpu(), want, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_feed_forward_part(name, model_and_plain):
    model, _, cfg, t, s = model_and_plain(name)
    h = torch.randn(13, s["H"])
    want = plain_qwen3.swiglu_mlp(h, t, "model.layers.0.")
    got = model.blocks[0].feed_forward.forward(h.cuda(), None)
    torch.testing.assert_close(got.cpu(), want, rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("name", ["A", "B"])
def test_block_arrangement(name, model_and_plain):
    from acvram_b200.parts import CacheView
    model, runner, cfg, t, s = model_and_plain(name)
    n = 19
    x = torch.randn(n, s["H"]) * 0.5
    want = plain_qwen3.decoder_layer(x, t, 0, s, torch.arange(n))
    ctx = ctx_for(runner, "a", [1] * n)
    k, v = runner.storage.pages(0)
    xs, delta = model.blocks[0].forward(x.cuda(), None, ctx, CacheView(0, True, k_pages=k, v_pages=v))
    torch.testing.assert_close((xs + delta).cpu(), want, rtol=2e-5, atol=2e-5)


def test_head_is_float32_and_tied(model_and_plain):
    model, _, cfg, t, s = model_and_plain("A", torch.bfloat16)
    assert model.head.weight.data_ptr() == model.embedding.data_ptr(), "a tied head shares the embedding's storage"
    h = (torch.randn(3, s["H"]) * 2).bfloat16()
    got = model.head(h.cuda(), out_dtype=torch.float32)
    assert got.dtype == torch.float32
    want = h.float() @ t["model.embed_tokens.weight"].T
    torch.testing.assert_close(got.cpu(), want, rtol=1e-5, atol=1e-5)


def test_kernels_refuse_cpu_tensors_and_unknown_types():
    from acvram_b200.kernels import KernelError, ops
    with pytest.raises(KernelError):
        ops.swiglu(torch.zeros(2, 8), torch.zeros(2, 4))
    with pytest.raises(KernelError):
        ops.swiglu(torch.zeros(2, 8, device="cuda", dtype=torch.float16), torch.zeros(2, 4, device="cuda", dtype=torch.float16))
    with pytest.raises(KernelError):   # head size beyond what the generic attention kernel takes
        q = torch.zeros(1, 3 * 512, device="cuda")
        pages = torch.zeros(1, 1, 16, 512, device="cuda")
        z = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.attention_generic(q, torch.zeros(1, 512, device="cuda"), pages, pages, z, z, z.view(1, 1), 1, 1, 512, 1.0)
