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


@pytest.mark.parametrize("name,dtype,window", [("A", "float32", 16), ("F", "bfloat16", 40), ("D", "bfloat16", 24)])
def test_window_layers_on_the_device(name, dtype, window, tiny_folders, plain_models):
    """A window on the second layer (a toy plan of the test's own): another cache group with pages given back as the
    window passes them, their block-table entries on the device set to "no page", and later pages of the same request
    taking the freed ones.  Portions and single tokens, two requests, against the plain layers."""
    import dataclasses

    import numpy as np

    import plain_qwen3
    from acvram_b200.engine.batch import StepEntry
    from acvram_b200.engine.runner import ModelRunner
    from acvram_b200.models import DecoderModel, plan_of_folder
    from acvram_b200.parts import Runtime
    from acvram_b200.weights import load_tensors
    from conftest import random_ids

    cfg, t = plain_models[name]
    _, plan = plan_of_folder(tiny_folders[name])
    layers = list(plan.layers)
    layers[1] = dataclasses.replace(layers[1], mixer=layers[1].mixer.with_params(window=window))
    plan = dataclasses.replace(plan, layers=tuple(layers))
    model = DecoderModel(plan)
    run_dtype = getattr(torch, dtype)
    model.load(load_tensors(tiny_folders[name], model.tensor_needs()), Runtime(torch.device("cuda:0"), run_dtype))
    assert len(model.cache_plan().groups) == 2
    page = 8
    pool = (60 + 2 * window) // page + 8                 # the windowed group's pool holds less than the requests' tokens
    runner = ModelRunner(model, page, [40, pool], 3)
    if run_dtype == torch.bfloat16:
        runner.enable_graphs()
    reqs = {"a": random_ids(cfg["vocab_size"], 150, 61), "b": random_ids(cfg["vocab_size"], 90, 62)}

    def plain(ids, dt):
        s = plain_qwen3.sizes(cfg)
        x = plain_qwen3.embed(t["model.embed_tokens.weight"], torch.tensor(ids), dt)
        positions = torch.arange(len(ids))
        for i in range(s["L"]):
            x = plain_qwen3.decoder_layer(x, t, i, s, positions, window if i == 1 else 0)
        return plain_qwen3.output_logits(x, t, s).numpy()

    ref = {k: plain(v, torch.float32) for k, v in reqs.items()}
    if dtype == "float32":
        bound = 2e-5 * max(1.0, max(float(np.abs(v).max()) for v in ref.values()))
    else:
        bound = 2.5 * max(float(np.abs(plain(v, torch.bfloat16) - ref[k]).max()) for k, v in reqs.items())
    at = {"a": 0, "b": 0}
    worst = 0.0
    schedule = [{"a": 37}, {"a": 2, "b": 30}, {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": 40, "b": 1}, {"a": 1, "b": 17},
                {"a": 1, "b": 1}, {"a": 1, "b": 1}, {"a": 60, "b": 1}, {"a": 1, "b": 30}] + [{"a": 1, "b": 1}] * 6
    for step in schedule:
        entries = []
        for k, n in step.items():
            n = min(n, len(reqs[k]) - at[k])
            if n > 0:
                entries.append(StepEntry(k, reqs[k][at[k]:at[k] + n], range(n)))
        lg = runner.step(entries).float().cpu().numpy()
        row = 0
        for e in entries:
            for i in range(len(e.tokens)):
                worst = max(worst, float(np.abs(lg[row] - ref[e.request][at[e.request] + i]).max()))
                row += 1
            at[e.request] += len(e.tokens)
    runner.check_status()
    assert worst <= bound, f"max |logit - plain| = {worst:.3e} (bound {bound:.3e})"
    full_free, window_free = runner.manager.free_pages()
    held = sum(-(-at[k] // page) for k in reqs)
    assert full_free == 40 - held and window_free >= pool - 2 * (window // page + 2), "the window's pages went back"
    for k in reqs:
        runner.release(k)
    runner.manager.check()
    assert runner.manager.free_pages() == [40, pool]
