"""Typed configuration of the ``LlamaForCausalLM`` architecture.

Every number the model needs is read from ``config.json``'s own keys; no size
or constant stands in code.  Keys, defaults and refusals follow the reference
(``models/llama/llama.py:59-95`` and ``models/blocks/rope.py:228-269``):

* ``head_dim`` defaults to ``hidden_size // num_attention_heads``;
* RoPE parameters live in ``rope_parameters`` or ``rope_scaling`` (the type under
  ``rope_type`` or ``type``), ``rope_theta`` inside that mapping or at top level,
  default 10000.0;
* a rope type other than ``default``/``llama3`` raises ``NotImplementedError``,
  a ``llama3`` mapping with a field missing raises ``ValueError``;
* ``attention_bias`` / ``mlp_bias`` must be false.

``max_position_embeddings`` is kept only as an optional upper bound that the
scheduler may check; position tables are computed from positions and have no
length.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .registry import ConfigError


@dataclass(frozen=True)
class Llama3RopeScaling:
    """The ``rope_type: "llama3"`` frequency rescale (reference
    ``models/blocks/rope.py:171-197``)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def __post_init__(self) -> None:
        if not self.factor > 0:
            raise ConfigError(f"llama3 rope factor must be positive, got {self.factor}")
        if not self.high_freq_factor > self.low_freq_factor:
            raise ConfigError(
                "llama3 rope needs high_freq_factor > low_freq_factor, got "
                f"{self.high_freq_factor} <= {self.low_freq_factor}"
            )
        if not self.original_max_position_embeddings > 0:
            raise ConfigError(
                "llama3 rope original_max_position_embeddings must be positive, got "
                f"{self.original_max_position_embeddings}"
            )


def read_rope_parameters(raw: Mapping[str, Any]) -> tuple[float, Llama3RopeScaling | None]:
    """``(rope_theta, llama3 scaling or None)`` from raw ``config.json`` keys."""
    params = raw.get("rope_parameters") or raw.get("rope_scaling") or {}
    if not isinstance(params, Mapping):
        raise ConfigError(f"rope_scaling must be an object, got {params!r}")
    if "rope_theta" in params:
        theta = float(params["rope_theta"])
    else:
        theta = float(raw.get("rope_theta") or 10000.0)
    rope_type = params.get("rope_type") or params.get("type") or "default"
    if rope_type == "default":
        return theta, None
    if rope_type == "llama3":
        try:
            scaling = Llama3RopeScaling(
                factor=float(params["factor"]),
                low_freq_factor=float(params["low_freq_factor"]),
                high_freq_factor=float(params["high_freq_factor"]),
                original_max_position_embeddings=int(params["original_max_position_embeddings"]),
            )
        except KeyError as missing:
            raise ConfigError(
                f"llama3 rope parameters are missing {missing}; got {sorted(params)}"
            ) from None
        return theta, scaling
    raise NotImplementedError(
        f"rope_type={rope_type!r} is not supported; only 'default' and 'llama3' are"
    )


def _required(raw: Mapping[str, Any], key: str, kind: type):
    if key not in raw or raw[key] is None:
        raise ConfigError(f"config.json lacks required key {key!r}")
    value = raw[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json key {key!r} must be an integer, got {value!r}")
        if value <= 0:
            raise ConfigError(f"config.json key {key!r} must be positive, got {value!r}")
        return value
    if kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json key {key!r} must be a number, got {value!r}")
        return float(value)
    return value


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    rope_scaling: Llama3RopeScaling | None = None
    max_position_embeddings: int | None = None
    architecture: str = field(default="LlamaForCausalLM")

    def __post_init__(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads != 0:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim % 2 != 0:
            raise ConfigError(f"head_dim must be even for rotary encoding, got {self.head_dim}")
        if not self.rms_norm_eps > 0:
            raise ConfigError(f"rms_norm_eps must be positive, got {self.rms_norm_eps}")

    @classmethod
    def from_json(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        """Parse the raw ``config.json`` mapping."""
        if raw.get("attention_bias"):
            raise NotImplementedError("LlamaForCausalLM with attention_bias=true is not supported")
        if raw.get("mlp_bias"):
            raise NotImplementedError("LlamaForCausalLM with mlp_bias=true is not supported")
        hidden = _required(raw, "hidden_size", int)
        heads = _required(raw, "num_attention_heads", int)
        head_dim = raw.get("head_dim") or hidden // heads
        theta, scaling = read_rope_parameters(raw)
        archs = raw.get("architectures") or ["LlamaForCausalLM"]
        max_pos = raw.get("max_position_embeddings")
        return cls(
            vocab_size=_required(raw, "vocab_size", int),
            hidden_size=hidden,
            intermediate_size=_required(raw, "intermediate_size", int),
            num_hidden_layers=_required(raw, "num_hidden_layers", int),
            num_attention_heads=heads,
            num_key_value_heads=int(raw.get("num_key_value_heads") or heads),
            head_dim=int(head_dim),
            rms_norm_eps=_required(raw, "rms_norm_eps", float),
            rope_theta=theta,
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            rope_scaling=scaling,
            max_position_embeddings=int(max_pos) if max_pos else None,
            architecture=str(archs[0]),
        )

    def to_json(self) -> dict[str, Any]:
        """The ``config.json`` mapping that parses back to this configuration."""
        raw: dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "llama",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "attention_bias": False,
            "mlp_bias": False,
            "hidden_act": "silu",
        }
        if self.rope_scaling is not None:
            s = self.rope_scaling
            raw["rope_scaling"] = {
                "rope_type": "llama3",
                "factor": s.factor,
                "low_freq_factor": s.low_freq_factor,
                "high_freq_factor": s.high_freq_factor,
                "original_max_position_embeddings": s.original_max_position_embeddings,
            }
        else:
            raw["rope_scaling"] = None
        if self.max_position_embeddings is not None:
            raw["max_position_embeddings"] = self.max_position_embeddings
        return raw
