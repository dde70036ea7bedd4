"""Typed configuration of Qwen3 dense (``Qwen3ForCausalLM``).

Every size and constant of the model comes from the keys of its ``config.json``.
Where a key is absent the default is the reference's own
(acvram/engine/config.py:891-906: hidden 4096, intermediate 11008, 32 layers,
32 heads, kv heads = heads, vocabulary 32000, 4096 positions, eps 1e-5 with the
fallback key ``norm_epsilon``, theta 10000, untied head; ``head_dim`` 0 means
hidden/heads, acvram/engine/config.py:177-179).  Nothing else in the package
holds a size.
"""

from __future__ import annotations

from dataclasses import dataclass, asdict
from typing import Any, Mapping

from .base import ConfigError, take_float, take_id_list, take_int


@dataclass(frozen=True)
class Qwen3Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    max_position_embeddings: int
    tie_word_embeddings: bool
    hidden_act: str = "silu"
    eos_token_id: tuple[int, ...] = ()
    bos_token_id: int | None = None

    architecture = "Qwen3ForCausalLM"
    model_type = "qwen3"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, cfg: Mapping[str, Any]) -> "Qwen3Config":
        heads = take_int(cfg, "num_attention_heads", 32)
        hidden = take_int(cfg, "hidden_size", 4096)
        head_dim = cfg.get("head_dim", 0) or 0
        if isinstance(head_dim, bool) or not isinstance(head_dim, int) or head_dim < 0:
            raise ConfigError(f"config key 'head_dim' must be a non-negative integer, got {head_dim!r}")
        if head_dim == 0:
            if hidden % heads:
                raise ConfigError(
                    f"'head_dim' is absent and hidden_size {hidden} is not a multiple of "
                    f"num_attention_heads {heads}")
            head_dim = hidden // heads
        eps_default = cfg.get("norm_epsilon", 1e-5)
        act = cfg.get("hidden_act") or cfg.get("hidden_activation") or "silu"
        bos = cfg.get("bos_token_id")
        self = cls(
            vocab_size=take_int(cfg, "vocab_size", 32000),
            hidden_size=hidden,
            intermediate_size=take_int(cfg, "intermediate_size", 11008),
            num_hidden_layers=take_int(cfg, "num_hidden_layers", 32),
            num_attention_heads=heads,
            num_key_value_heads=take_int(cfg, "num_key_value_heads", heads),
            head_dim=head_dim,
            rms_norm_eps=take_float(cfg, "rms_norm_eps", eps_default),
            rope_theta=take_float(cfg, "rope_theta", 10000.0),
            max_position_embeddings=take_int(cfg, "max_position_embeddings", 4096),
            tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            hidden_act=str(act),
            eos_token_id=take_id_list(cfg, "eos_token_id"),
            bos_token_id=bos if isinstance(bos, int) and not isinstance(bos, bool) else None,
        )
        self._check_unsupported(cfg)
        self.validate()
        return self

    @staticmethod
    def _check_unsupported(cfg: Mapping[str, Any]) -> None:
        scaling = cfg.get("rope_scaling")
        if scaling not in (None, {}):
            kind = scaling.get("rope_type") or scaling.get("type") if isinstance(scaling, dict) else scaling
            if kind not in (None, "default"):
                raise ConfigError(
                    f"config key 'rope_scaling' = {scaling!r}: only unscaled rotary positions are built")
        if cfg.get("use_sliding_window"):
            raise ConfigError(
                "config key 'use_sliding_window' is true: Qwen3 dense runs with full attention here "
                "(the reference ignores the window keys for this architecture)")
        if cfg.get("attention_bias"):
            raise ConfigError("config key 'attention_bias' is true: Qwen3 dense has no biases")

    def validate(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}")
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary positions")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act '{self.hidden_act}' is not built; Qwen3 uses 'silu'")
        for tok in self.eos_token_id:
            if not 0 <= tok < self.vocab_size:
                raise ConfigError(f"eos_token_id {tok} is outside the vocabulary of {self.vocab_size}")

    # ------------------------------------------------------------------ derived
    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict[str, Any]:
        out = asdict(self)
        eos = list(self.eos_token_id)
        out["eos_token_id"] = eos[0] if len(eos) == 1 else (eos or None)
        out["architectures"] = [self.architecture]
        out["model_type"] = self.model_type
        return out
