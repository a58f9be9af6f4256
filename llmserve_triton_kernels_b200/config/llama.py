"""Typed configuration of the Llama architecture, read from its own config.json keys.

Parity: the reference's ``ModelConfig.from_hf_dict`` (src/llmserve/config.py:39-61) reads the
same keys with the same defaults; ``head_dim`` is derived as ``hidden_size // num_attention_heads``
(src/llmserve/config.py:22-24) and any non-default ``rope_scaling`` is refused
(src/llmserve/config.py:41-46).  Nothing here is a size of a particular checkpoint: every
number comes from the dictionary.
"""

from __future__ import annotations

from dataclasses import asdict, dataclass


class ConfigError(ValueError):
    """A config.json that this engine cannot run, with the offending key named."""


def _require(d: dict, key: str, kind=int):
    if key not in d:
        raise ConfigError(f"config.json is missing the required key {key!r}")
    value = d[key]
    if kind is int and (isinstance(value, bool) or not isinstance(value, int)):
        raise ConfigError(f"config.json key {key!r} must be an integer, got {value!r}")
    return value


@dataclass(frozen=True)
class LlamaConfig:
    """The numbers a Llama decoder is built from (keys of its config.json in brackets)."""

    vocab_size: int  # [vocab_size]
    hidden_size: int  # [hidden_size]
    intermediate_size: int  # [intermediate_size]
    num_hidden_layers: int  # [num_hidden_layers]
    num_attention_heads: int  # [num_attention_heads]
    num_key_value_heads: int  # [num_key_value_heads], default: num_attention_heads
    max_position_embeddings: int  # [max_position_embeddings], a length guard and table size
    rope_theta: float  # [rope_theta] or [rope_parameters.rope_theta]
    rms_norm_eps: float  # [rms_norm_eps]
    tie_word_embeddings: bool  # [tie_word_embeddings]

    architecture = "LlamaForCausalLM"

    def __post_init__(self) -> None:
        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "max_position_embeddings",
        ):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.hidden_size % self.num_attention_heads:
            raise ConfigError(
                f"hidden_size {self.hidden_size} is not divisible by num_attention_heads "
                f"{self.num_attention_heads}"
            )
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for rotary positions")
        if self.head_dim > 256:
            raise ConfigError(
                f"hidden_size {self.hidden_size} / num_attention_heads {self.num_attention_heads} gives head_dim "
                f"{self.head_dim}; the attention kernels take head sizes up to 256"
            )
        if not self.rms_norm_eps > 0 or not self.rope_theta > 0:
            raise ConfigError("rms_norm_eps and rope_theta must be positive")

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @classmethod
    def from_dict(cls, d: dict) -> "LlamaConfig":
        scaling = d.get("rope_scaling")
        if scaling and scaling.get("rope_type", scaling.get("type")) not in (None, "default"):
            raise ConfigError(
                f"rope_scaling={scaling!r} is not supported: this engine runs Llama with unscaled "
                "rotary positions (TinyLlama, Llama-2; not Llama-3.1 and later)"
            )
        rope_theta = d.get("rope_theta") or (d.get("rope_parameters") or {}).get("rope_theta", 10000.0)
        heads = _require(d, "num_attention_heads")
        hidden = _require(d, "hidden_size")
        if d.get("head_dim") is not None and heads > 0 and d["head_dim"] != hidden // heads:
            raise ConfigError(
                f"head_dim {d['head_dim']} differs from hidden_size // num_attention_heads = "
                f"{hidden // heads}; this architecture derives it"
            )
        if d.get("hidden_act", "silu") != "silu":
            raise ConfigError(f"hidden_act {d['hidden_act']!r} is not supported (the feed-forward is SwiGLU)")
        for key in ("attention_bias", "mlp_bias"):
            if d.get(key):
                raise ConfigError(f"{key}=true is not supported (Llama projections carry no bias)")
        return cls(
            vocab_size=_require(d, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_require(d, "intermediate_size"),
            num_hidden_layers=_require(d, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=int(d.get("num_key_value_heads") or heads),
            max_position_embeddings=int(d.get("max_position_embeddings", 2048)),
            rope_theta=float(rope_theta),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
        )

    def to_dict(self) -> dict:
        """The config.json this configuration is read back from."""
        d = asdict(self)
        d["architectures"] = [self.architecture]
        d["model_type"] = "llama"
        d["hidden_act"] = "silu"
        return d
