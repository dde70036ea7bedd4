"""Models: the generic decoder and the plans of the built architectures."""

from __future__ import annotations

import os

import torch

from ..config import family_of, read_config_json
from ..parts import ModelPlan, Runtime
from ..weights import load_tensors, random_tensors
from . import qwen3  # noqa: F401  (registers Qwen3ForCausalLM)
from .decoder import DecoderModel

__all__ = ["DecoderModel", "build_from_folder", "build_random", "needs_of_plan", "plan_of_folder"]


def needs_of_plan(plan: ModelPlan):
    return DecoderModel(plan).tensor_needs()


def plan_of_folder(folder: str | os.PathLike):
    cfg = read_config_json(folder)
    family = family_of(cfg)
    config = family.config_cls.from_dict(cfg)
    return config, family.build_plan(config)


def build_from_folder(folder: str | os.PathLike, dtype: torch.dtype, device="cuda:0"):
    """(config, model) from config.json + safetensors; the model class follows config.json."""
    config, plan = plan_of_folder(folder)
    model = DecoderModel(plan)
    tensors = load_tensors(folder, model.tensor_needs(), device="cpu")
    model.load(tensors, Runtime(torch.device(device), dtype))
    return config, model


def build_random(config, seed: int, dtype: torch.dtype, device="cuda:0"):
    """A model with seeded random weights made on the device (no file in between)."""
    plan = family_of(config.to_dict()).build_plan(config)
    model = DecoderModel(plan)
    rt = Runtime(torch.device(device), dtype)
    tensors = dict(random_tensors(model.tensor_needs(), seed, rt.device, torch.bfloat16))
    model.load(tensors, rt)
    return model
