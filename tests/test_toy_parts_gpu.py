"""Parts that are not this architecture's, defined here and registered without a change to the package:
a mixer with per-request state of fixed size, another position encoding, a feed-forward with routing.
They are toys to show the interfaces; they are no model of anyone's."""

from __future__ import annotations

import dataclasses

import pytest
import torch

import plain_qwen3 as P
from conftest import random_ids, tiny_config

pytestmark = pytest.mark.gpu


def register_toys():
    from acvram_b200.cache import StateNeed
    from acvram_b200.parts import FeedForward, Mixer, PositionEncoding, register
    from acvram_b200.weights import TensorNeed

    @register("mixer", "toy_decay")
    class DecayMixer(Mixer):
        """state = decay * state + x_t (per request, carried across steps); out_t = state @ W^T."""

        capturable = False      # its loop reads the state slots on the host

        def __init__(self, hidden_size, decay):
            self.h, self.decay = hidden_size, float(decay)

        def cache_need(self):
            return StateNeed((self.h,), "float32")

        def tensor_needs(self):
            return {"toy.w.weight": TensorNeed((self.h, self.h))}

        def load(self, tensors, rt):
            self.w = tensors["toy.w.weight"].to(rt.device, torch.float32)
            self.dtype = rt.dtype

        def forward(self, h, ctx, cache):
            out = torch.empty_like(h, dtype=torch.float32)
            slots = ctx.state_slots[cache.group].tolist()
            start = 0
            for slot, n in zip(slots, ctx.q_lens):
                s = cache.state[slot]
                for i in range(start, start + n):
                    s.mul_(self.decay).add_(h[i].float())
                    out[i] = s
                start += n
            return (out @ self.w.T).to(h.dtype)

    @register("mixer", "toy_sum")
    class SumMixer(Mixer):
        """state = state + x_t; out_t = state @ W^T: the same kind of state, kept with device operations only
        (the slots are never read on the host), so that a step with it can be captured in a CUDA graph."""

        def __init__(self, hidden_size):
            self.h = hidden_size

        def cache_need(self):
            return StateNeed((self.h,), "float32")

        def tensor_needs(self):
            return {"toy.w.weight": TensorNeed((self.h, self.h))}

        def load(self, tensors, rt):
            self.w = tensors["toy.w.weight"].to(rt.device, torch.float32)

        def forward(self, h, ctx, cache):
            slots = ctx.state_slots[cache.group].long()
            seq, cu = ctx.seq_of_token.long(), ctx.cu_q.long()
            run = torch.cat((torch.zeros(1, self.h, device=h.device), torch.cumsum(h.float(), 0)))
            out = run[1:] - run[cu[seq]] + cache.state[slots[seq]]
            cache.state.index_add_(0, slots, run[cu[1:]] - run[cu[:-1]])
            return (out @ self.w.T).to(h.dtype)

    @register("position", "toy_position_scale")
    class PositionScale(PositionEncoding):
        """q and k of the token at position p are multiplied by 1 + strength * (p mod 7)."""

        def __init__(self, hidden_size, strength):
            self.strength = float(strength)

        def apply(self, q, k, ctx):
            f = (1.0 + self.strength * (ctx.positions % 7).float()).to(q.dtype)[:, None, None]
            q.mul_(f)
            k.mul_(f)

    @register("feed_forward", "toy_routed")
    class RoutedFF(FeedForward):
        """Two experts; each token goes to the expert with the larger router logit (router in float32)."""

        def __init__(self, hidden_size, width):
            self.h, self.width = hidden_size, width

        def tensor_needs(self):
            n = {"toy_router.weight": TensorNeed((2, self.h))}
            for e in range(2):
                n[f"toy_experts.{e}.up.weight"] = TensorNeed((self.width, self.h))
                n[f"toy_experts.{e}.down.weight"] = TensorNeed((self.h, self.width))
            return n

        def load(self, tensors, rt):
            self.t = {k: v.to(rt.device, torch.float32) for k, v in tensors.items()}

        def forward(self, h, ctx):
            # both experts run on every token and the router picks the result: no shape depends on the data, so
            # the host never has to read the choice (a toy: a real routed feed-forward would permute the tokens)
            x = h.float()
            choice = (x @ self.t["toy_router.weight"].T).argmax(-1)
            outs = [torch.relu(x @ self.t[f"toy_experts.{e}.up.weight"].T) @ self.t[f"toy_experts.{e}.down.weight"].T
                    for e in range(2)]
            return torch.where((choice == 0)[:, None], outs[0], outs[1]).to(h.dtype)


def toy_plan(cfg, state_mixer=("toy_decay", {"decay": 0.9})):
    """Layer 0: attention with the toy position encoding and the routed feed-forward; layer 1: the stateful
    mixer with the usual feed-forward; layer 2: attention as the architecture has it, but with biases on all
    its projections and on the feed-forward's."""
    from acvram_b200.models.qwen3 import qwen3_plan
    from acvram_b200.parts import PartSpec
    plan = qwen3_plan(cfg)
    layers = list(plan.layers)
    layers[0] = dataclasses.replace(
        layers[0], mixer=layers[0].mixer.with_params(position=PartSpec("toy_position_scale", {"strength": 0.05})),
        feed_forward=PartSpec("toy_routed", {"width": 40}))
    layers[1] = dataclasses.replace(layers[1], mixer=PartSpec(*state_mixer))
    layers[2] = dataclasses.replace(layers[2], mixer=layers[2].mixer.with_params(bias=True),
                                    feed_forward=layers[2].feed_forward.with_params(bias=True))
    return dataclasses.replace(plan, architecture="ToyForTests", layers=tuple(layers))


def plain_toy_logits(cfg: dict, t: dict, ids, state_mixer="toy_decay", dtype=torch.float32) -> torch.Tensor:
    """The toy model restated plainly, whole sequence, no cache: the architecture's parts come from the plain
    implementation, the toys are written out again here from their definitions."""
    s = P.sizes(cfg)
    ids = torch.as_tensor(ids, dtype=torch.long)
    T = ids.numel()
    pos = torch.arange(T)
    x = P.embed(t["model.embed_tokens.weight"], ids, dtype)
    # layer 0: attention whose q and k are scaled by 1 + 0.05 (p mod 7) after the norm, no rotation; routed feed-forward
    p = "model.layers.0."
    h = P.rms_norm(x, t[p + "input_layernorm.weight"], s["eps"])
    q = P.proj(h, t, p + "self_attn.q_proj.").view(T, s["NH"], s["D"])
    k = P.proj(h, t, p + "self_attn.k_proj.").view(T, s["NKV"], s["D"])
    v = P.proj(h, t, p + "self_attn.v_proj.").view(T, s["NKV"], s["D"])
    ones, zeros = torch.ones(T, s["D"]), torch.zeros(T, s["D"])
    q = P.qk_norm_rotary(q, t[p + "self_attn.q_norm.weight"], s["eps"], ones, zeros)
    k = P.qk_norm_rotary(k, t[p + "self_attn.k_norm.weight"], s["eps"], ones, zeros)
    f = (1.0 + 0.05 * (pos % 7).float()).to(dtype)[:, None, None]
    o = P.causal_attention(q * f, k * f, v, s["D"] ** -0.5)
    x = P.residual_add(x, P.proj(o.reshape(T, -1), t, p + "self_attn.o_proj."))
    h = P.rms_norm(x, t[p + "post_attention_layernorm.weight"], s["eps"]).float()
    choice = (h @ t[p + "toy_router.weight"].T).argmax(-1)
    y = torch.zeros_like(h)
    for e in range(2):
        m = choice == e
        y[m] = torch.relu(h[m] @ t[p + f"toy_experts.{e}.up.weight"].T) @ t[p + f"toy_experts.{e}.down.weight"].T
    x = P.residual_add(x, y.to(dtype))
    # layer 1: the mixer with a state (a decaying or a plain running sum), then the usual feed-forward
    p = "model.layers.1."
    h = P.rms_norm(x, t[p + "input_layernorm.weight"], s["eps"]).float()
    state, outs = torch.zeros(s["H"]), []
    for i in range(T):
        state = (0.9 * state if state_mixer == "toy_decay" else state) + h[i]
        outs.append(state)
    x = P.residual_add(x, (torch.stack(outs) @ t[p + "toy.w.weight"].T).to(dtype))
    h = P.rms_norm(x, t[p + "post_attention_layernorm.weight"], s["eps"])
    x = P.residual_add(x, P.swiglu_mlp(h, t, p))
    # layer 2: the architecture's own layer (its tensors include biases, which the plain parts add where they find them)
    x = P.decoder_layer(x, t, 2, s, pos)
    return P.output_logits(x, t, s)


def test_toy_parts_register_build_and_step(tmp_path):
    from acvram_b200.config import REGISTRY, Qwen3Config, register_architecture
    from acvram_b200.engine.batch import StepEntry
    from acvram_b200.engine.runner import ModelRunner
    from acvram_b200.models import build_from_folder
    from acvram_b200.weights import write_random_model

    register_toys()

    class ToyConfig(Qwen3Config):
        architecture = "ToyForTests"

    register_architecture("ToyForTests", ToyConfig, toy_plan)
    try:
        cfg = ToyConfig(**dataclasses.asdict(tiny_config("B")))
        write_random_model(cfg, tmp_path, seed=9)
        _, model = build_from_folder(tmp_path, torch.float32, "cuda:0")
        cplan = model.cache_plan()
        kinds = [g.kind for g in cplan.groups]
        assert kinds == ["paged", "state"] and cplan.slots_per_group == [2, 1]
        assert model.uncapturable_parts() == ["toy_decay"]
        assert model.blocks[2].mixer.qkv.bias is not None and model.blocks[2].feed_forward.down.bias is not None
        assert model.blocks[0].mixer.qkv.bias is None, "a bias is read only where the plan asks or the file has one"

        runner = ModelRunner(model, 8, 32, 3)
        a = random_ids(cfg.vocab_size, 37, 1)
        b = random_ids(cfg.vocab_size, 20, 2)
        whole_a = runner.step([StepEntry("wa", a, range(37))])
        whole_b = runner.step([StepEntry("wb", b, range(20))])
        runner.release("wa"); runner.release("wb")

        # the engine's toy model is the toys' plain restatement ...
        plain_cfg, plain_t = P.read_folder(str(tmp_path))
        torch.testing.assert_close(whole_a.cpu(), plain_toy_logits(plain_cfg, plain_t, a), rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(whole_b.cpu(), plain_toy_logits(plain_cfg, plain_t, b), rtol=2e-5, atol=2e-5)
        # ... and the toys matter: with another rule for the state (the other toy's) the logits are far from it
        assert (plain_toy_logits(plain_cfg, plain_t, a, "toy_sum") - whole_a.cpu()).abs().max() > 0.05

        # portions of a beside b (whole, then its tokens one by one would be the same state hand-over)
        got_a, got_b = [], []
        lg = runner.step([StepEntry("a", a[:11], range(11)), StepEntry("b", b[:9], range(9))])
        got_a.append(lg[:11]); got_b.append(lg[11:])
        lg = runner.step([StepEntry("b", b[9:10], [0]), StepEntry("a", a[11:13], range(2))])
        got_b.append(lg[:1]); got_a.append(lg[1:])
        lg = runner.step([StepEntry("a", a[13:], range(24)), StepEntry("b", b[10:], range(10))])
        got_a.append(lg[:24]); got_b.append(lg[24:])
        torch.testing.assert_close(torch.cat(got_a), whole_a, rtol=2e-5, atol=2e-5)
        torch.testing.assert_close(torch.cat(got_b), whole_b, rtol=2e-5, atol=2e-5)

        # a state slot is zeroed when it is given to a new request
        runner.release("a"); runner.release("b")
        again = runner.step([StepEntry("c", a, range(37))])
        torch.testing.assert_close(again, whole_a, rtol=2e-5, atol=2e-5)
        runner.release("c")
        runner.manager.check()

    finally:
        REGISTRY.pop("ToyForTests", None)


def test_a_state_of_fixed_size_inside_a_captured_decode_step(tmp_path):
    """bfloat16, decode steps replayed from CUDA graphs, with a mixer that keeps a state of fixed size by device
    operations only: the state slots travel with every step, padding rows work on the slot that belongs to nobody,
    a slot is zeroed when a new request takes it.  Compared with the toys' plain restatement."""
    from acvram_b200.config import REGISTRY, Qwen3Config, register_architecture
    from acvram_b200.engine.batch import StepEntry
    from acvram_b200.engine.runner import ModelRunner
    from acvram_b200.models import build_from_folder
    from acvram_b200.weights import write_random_model

    register_toys()

    class ToyConfig(Qwen3Config):
        architecture = "ToyForTests"

    register_architecture("ToyForTests", ToyConfig, lambda cfg: toy_plan(cfg, ("toy_sum", {})))
    try:
        cfg = ToyConfig(**dataclasses.asdict(tiny_config("D")))      # heads of 64: the tensor-core attention kernels
        cfg = dataclasses.replace(cfg, num_hidden_layers=3)
        write_random_model(cfg, tmp_path, seed=10)
        plain_cfg, plain_t = P.read_folder(str(tmp_path))
        _, model = build_from_folder(tmp_path, torch.bfloat16, "cuda:0")
        assert model.uncapturable_parts() == []
        runner = ModelRunner(model, 16, 32, 4)
        runner.enable_graphs()
        reqs = {f"r{i}": random_ids(cfg.vocab_size, n, 20 + i) for i, n in enumerate((30, 9, 17))}
        refs = {k: plain_toy_logits(plain_cfg, plain_t, v, "toy_sum") for k, v in reqs.items()}
        yard = max(float((plain_toy_logits(plain_cfg, plain_t, v, "toy_sum", torch.bfloat16) - refs[k]).abs().max())
                   for k, v in reqs.items())
        tail = 6
        runner.step([StepEntry(k, v[:-tail], ()) for k, v in reqs.items()])
        worst = 0.0
        for i in range(tail, 0, -1):
            lg = runner.step([StepEntry(k, v[len(v) - i:len(v) - i + 1], (0,)) for k, v in reqs.items()])
            for row, (k, v) in zip(lg, reqs.items()):
                worst = max(worst, float((row.float().cpu() - refs[k][len(v) - i]).abs().max()))
        assert runner.graphs.replays >= tail - 1 and runner.graphs.disabled_reason is None
        assert worst <= 2.5 * yard, f"{worst:.3e} against a bfloat16 yardstick of {yard:.3e}"
        # a new request in a slot that was used: its state starts at zero (three live requests pad the batch to four rows)
        runner.release("r1")
        again = runner.step([StepEntry("n", reqs["r1"], range(9))])
        assert float((again.float().cpu() - refs["r1"]).abs().max()) <= 2.5 * yard
        runner.check_status()
    finally:
        REGISTRY.pop("ToyForTests", None)
