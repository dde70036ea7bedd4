"""Qwen3 dense as a plan of parts.

Pre-norm decoder; grouped-query attention with per-head RMS norm of q and k
before rotary positions over the whole head; SwiGLU feed-forward; RMS norms with
one eps; no biases; full attention in every layer; the output head is its own
matrix or the embedding (acvram/engine/model.py:1-15 and the generic "llama" path
it runs for ``Qwen3ForCausalLM``, acvram/engine/config.py:644).
"""

from __future__ import annotations

from ..config.qwen3 import Qwen3Config
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, default_schedule


def qwen3_plan(cfg: Qwen3Config) -> ModelPlan:
    norm = PartSpec("rmsnorm", {"eps": cfg.rms_norm_eps})
    position = PartSpec("rotary", {"dim": cfg.head_dim, "theta": cfg.rope_theta,
                                   "max_positions": cfg.max_position_embeddings})
    mixer = PartSpec("attention", {
        "num_heads": cfg.num_attention_heads, "num_kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
        "position": position, "qk_norm_eps": cfg.rms_norm_eps, "window": 0})
    feed_forward = PartSpec("swiglu", {"intermediate_size": cfg.intermediate_size})
    layers = tuple(LayerSpec(f"model.layers.{i}.", "prenorm", mixer, feed_forward, norm)
                   for i in range(cfg.num_hidden_layers))
    return ModelPlan(
        architecture=cfg.architecture, hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings, layers=layers, schedule=default_schedule(cfg.num_hidden_layers),
        final_norm=norm, tied_head=cfg.tie_word_embeddings, eos_token_ids=cfg.eos_token_id)


register_architecture("Qwen3ForCausalLM", Qwen3Config, qwen3_plan)
