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


LLAMA3_FIELDS = (
    ("factor", float),
    ("low_freq_factor", float),
    ("high_freq_factor", float),
    ("original_max_position_embeddings", int),
)


@dataclass(frozen=True)
class Llama3RopeScaling:
    """The four numbers of a ``"llama3"`` rotary rescale: frequencies whose wavelength is
    longer than ``original_max_position_embeddings / low_freq_factor`` are divided by
    ``factor``, those shorter than ``... / high_freq_factor`` are kept, the band between is
    blended (what the numbers mean: reference ``models/blocks/rope.py:200-225``)."""

    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    def problems(self) -> list[str]:
        """Why these numbers cannot describe a rescale (empty: they can)."""
        found = []
        if not self.factor > 0:
            found.append(f"factor={self.factor} is not positive")
        if not self.low_freq_factor < self.high_freq_factor:
            found.append(f"low_freq_factor={self.low_freq_factor} is not below "
                         f"high_freq_factor={self.high_freq_factor}")
        if not self.original_max_position_embeddings > 0:
            found.append(f"original_max_position_embeddings={self.original_max_position_embeddings} "
                         "is not positive")
        return found

    def __post_init__(self) -> None:
        found = self.problems()
        if found:
            raise ConfigError("bad llama3 rope scaling: " + "; ".join(found))


def _llama3_from(section: Mapping[str, Any]) -> Llama3RopeScaling:
    absent = [key for key, _ in LLAMA3_FIELDS if section.get(key) is None]
    if absent:
        raise ConfigError(f"a llama3 rope scaling needs {', '.join(absent)}; config.json gives only "
                          f"{', '.join(sorted(section)) or 'nothing'}")
    return Llama3RopeScaling(**{key: kind(section[key]) for key, kind in LLAMA3_FIELDS})


# rope type (as config.json spells it) -> how its section becomes a scaling (None: no rescale)
ROPE_TYPES = {
    "default": lambda section: None,
    "llama3": _llama3_from,
}


def read_rope_parameters(raw: Mapping[str, Any]) -> tuple[float, Llama3RopeScaling | None]:
    """``(rope_theta, scaling or None)``.  The rotary settings sit in a section named
    ``rope_parameters`` (newer files) or ``rope_scaling``; its type is spelled ``rope_type`` or
    ``type``; ``rope_theta`` may sit inside the section or at the top level (the reference
    reads the same places, ``models/blocks/rope.py:228-269``)."""
    section: Any = {}
    for name in ("rope_parameters", "rope_scaling"):
        if raw.get(name):
            section = raw[name]
            break
    if not isinstance(section, Mapping):
        raise ConfigError(f"the rope section of config.json must be an object, got {section!r}")
    theta = section.get("rope_theta", raw.get("rope_theta"))
    kind = section.get("rope_type") or section.get("type") or "default"
    if kind not in ROPE_TYPES:
        raise NotImplementedError(f"rope type {kind!r}: this engine knows {sorted(ROPE_TYPES)}")
    return float(theta or 10000.0), ROPE_TYPES[kind](section)


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
