"""Random-weights mode: write a model folder from a configuration and a seed.

``write_random_model(raw_config, out_dir, seed)`` builds the architecture named by the
configuration (without touching a GPU), asks it which tensors it needs, draws each one
from a counter-based generator keyed by ``(seed, tensor name)`` with the element index as
the counter, and writes ``config.json`` and ``model.safetensors``.  Matrices and embeddings
are N(0, ``std``); norm gains are ``1 + N(0, gain_std)``.  Values are drawn in float64,
rounded to float32 and stored in ``store_dtype`` (bfloat16 by default, so that a bfloat16
engine, a float32 engine and a plain fp32 implementation all see exactly the same numbers).

*The same numbers on every device.*  An element's value depends on nothing but the seed, the
tensor's name and the element's index, and it is computed with integer arithmetic and with
float64 additions, multiplications and divisions only, each a separate, correctly rounded
operation: the logarithm, the square root and the sine of the Box-Muller transform are
evaluated by their own short series and iterations here instead of by a math library, whose
results differ between a CPU and a GPU in the last bit.  So a tensor drawn on a GPU (a
benchmark's 16 GB of weights never exist on the host) is bit for bit the tensor the CPU
draws, and a plain implementation on the CPU can be handed weights made on the device.

The reference has no such mode (its tests overwrite ``nn.Module`` defaults by hand,
``tests/unit/models/llama/test_llama_rope_scaling.py:83-92``).
"""

from __future__ import annotations

import hashlib
import json
import math
import os
from typing import Any, Mapping

import torch

from ..config.registry import load_config
from ..parts.model import DecoderModel
from .safetensors_io import write_safetensors

_MASK64 = (1 << 64) - 1
_CHUNK = 1 << 22          # elements drawn at a time on the CPU (bounds the temporaries: a few hundred MB)
_CHUNK_CUDA = 1 << 24     # on a GPU: fewer, larger launches


def tensor_seed(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFF_FFFF_FFFF_FFFF


def _signed(x: int) -> int:
    """A 64-bit pattern as the int64 that holds it."""
    x &= _MASK64
    return x - (1 << 64) if x >> 63 else x


def _shr(z: torch.Tensor, n: int) -> torch.Tensor:
    """Logical shift right of int64 bit patterns."""
    return (z >> n) & ((1 << (64 - n)) - 1)


_GAMMA = 0x9E3779B97F4A7C15
_MIX1 = 0xBF58476D1CE4E5B9
_MIX2 = 0x94D049BB133111EB


def hash_bits(key: int, index: torch.Tensor) -> torch.Tensor:
    """64 well-mixed bits per element: the counter ``key + (index + 1) * gamma`` pushed through
    two multiply-xorshift rounds (all arithmetic modulo 2^64, on int64 bit patterns)."""
    z = (index + 1) * _signed(_GAMMA) + _signed(key)
    z = (z ^ _shr(z, 30)) * _signed(_MIX1)
    z = (z ^ _shr(z, 27)) * _signed(_MIX2)
    return z ^ _shr(z, 31)


def hash_bits_exact(key: int, index: int) -> int:
    """The same function on Python integers (tests compare the tensor version with it)."""
    z = ((index + 1) * _GAMMA + key) & _MASK64
    z = ((z ^ (z >> 30)) * _MIX1) & _MASK64
    z = ((z ^ (z >> 27)) * _MIX2) & _MASK64
    return z ^ (z >> 31)


_LN2 = math.log(2.0)
_SQRT2 = math.sqrt(2.0)
_LOG_TERMS = 9            # 2 s (1 + s^2/3 + ... + s^16/17): |s| <= 0.1716, remainder below 1e-15
_SIN_TERMS = 11           # x - x^3/3! + ... - x^21/21!: x <= pi/2, remainder below 1e-15


def _log_of(x: torch.Tensor) -> torch.Tensor:
    """Natural logarithm of positive float64 numbers from exact operations only: the exponent
    and the mantissa are taken from the bit pattern, the mantissa's logarithm is the series
    ``2 atanh((m - 1) / (m + 1))``."""
    bits = x.view(torch.int64)
    e = ((bits >> 52) & 0x7FF) - 1023
    m = ((bits & ((1 << 52) - 1)) | (1023 << 52)).view(torch.float64)       # in [1, 2)
    high = m > _SQRT2
    m = torch.where(high, m * 0.5, m)                                        # in [0.7071, 1.4143)
    e = torch.where(high, e + 1, e)
    s = (m - 1.0) / (m + 1.0)
    s2 = s * s
    acc = torch.full_like(s, 1.0 / (2 * _LOG_TERMS - 1))
    for k in range(_LOG_TERMS - 2, -1, -1):
        acc = acc * s2 + 1.0 / (2 * k + 1)
    return e.to(torch.float64) * _LN2 + 2.0 * s * acc


def _sqrt_of(x: torch.Tensor) -> torch.Tensor:
    """Square root of positive float64 numbers by Newton's iteration from a guess made on the
    bit pattern (halving the exponent): divisions, additions and halvings only, so every
    device takes the same steps to the same bits.  (A library square root is not used: the
    CPU's and the GPU's were seen to differ in the last bit.)"""
    y = ((x.view(torch.int64) >> 1) + (1023 << 51)).view(torch.float64)       # within a few percent
    for _ in range(6):
        y = (y + x / y) * 0.5
    return y


def _sin_quarter(x: torch.Tensor) -> torch.Tensor:
    """``sin x`` for ``0 <= x <= pi / 2`` as its Taylor polynomial (exact operations only)."""
    x2 = x * x
    acc = torch.full_like(x, (-1.0) ** (_SIN_TERMS - 1) / math.factorial(2 * _SIN_TERMS - 1))
    for k in range(_SIN_TERMS - 2, -1, -1):
        acc = acc * x2 + (-1.0) ** k / math.factorial(2 * k + 1)
    return x * acc


def standard_normal(key: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """Elements ``start .. start + count - 1`` of the N(0, 1) stream of ``key``, float64.

    Box-Muller on the two halves of ``hash_bits``: ``sqrt(-2 ln u) cos(2 pi t)`` with
    ``u = (high half + 1/2) / 2^32`` and ``t = low half / 2^32``; the cosine is taken as a
    sine a quarter turn further, folded into the first quadrant on the integer."""
    index = torch.arange(start, start + count, dtype=torch.int64, device=device)
    z = hash_bits(key, index)
    hi = _shr(z, 32)
    lo = z & 0xFFFF_FFFF
    log_u = _log_of(hi.to(torch.float64) + 0.5) - 32.0 * _LN2
    radius = _sqrt_of(log_u * -2.0)
    turn = (lo + (1 << 30)) & 0xFFFF_FFFF            # a quarter turn further: cos -> sin
    quadrant = turn >> 30
    within = turn & ((1 << 30) - 1)
    folded = torch.where((quadrant & 1) == 1, (1 << 30) - within, within)
    angle = folded.to(torch.float64) * (math.pi / 2.0 / (1 << 30))
    sign = (1 - (quadrant & 2)).to(torch.float64)
    return radius * (sign * _sin_quarter(angle))


def random_tensor(seed: int, name: str, shape, role: str, *, std: float, gain_std: float,
                  device="cpu", dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """The tensor ``name`` of the model seeded with ``seed``: N(0, ``std``), or
    ``1 + N(0, gain_std)`` for a norm's gain; the same values on every device.  Computed in
    float64, rounded once to float32 and then to ``dtype``."""
    key = tensor_seed(seed, name)
    shape = tuple(int(n) for n in shape)
    total = 1
    for n in shape:
        total *= n
    out = torch.empty(total, dtype=dtype, device=device)
    chunk = _CHUNK_CUDA if torch.device(device).type == "cuda" else _CHUNK
    for start in range(0, total, chunk):
        count = min(chunk, total - start)
        z = standard_normal(key, start, count, device)
        z = z * gain_std + 1.0 if role == "gain" else z * std
        out[start:start + count] = z.to(torch.float32).to(dtype)
    return out.view(shape)


def std_of(name: str, std: float, std_overrides: Mapping[str, float] | None) -> float:
    for key, value in (std_overrides or {}).items():
        if key in name:
            std = value
    return std


def bind_random(model: DecoderModel, seed: int, dtype: torch.dtype, device, *, std: float = 0.02,
                gain_std: float = 0.1, std_overrides: Mapping[str, float] | None = None,
                store_dtype: torch.dtype = torch.bfloat16) -> None:
    """Give ``model`` the weights ``write_random_model`` would write for ``seed``, drawn on
    ``device`` one part at a time (nothing goes through a file or the host, and nothing but
    the part being bound exists twice)."""
    from .loader import TensorSource, to_engine_dtype

    decls = {e.name: e.decl for e in model.expected_tensors()}

    def draw(name: str) -> torch.Tensor:
        decl = decls[name]
        t = random_tensor(seed, name, decl.shape, decl.role, std=std_of(name, std, std_overrides),
                          gain_std=gain_std, device=device, dtype=store_dtype)
        return to_engine_dtype(t, dtype)

    model.bind(TensorSource(draw), dtype, torch.device(device))


def random_state_dict(raw_config: Mapping[str, Any], seed: int, *, std: float = 0.02,
                      gain_std: float = 0.1, std_overrides: Mapping[str, float] | None = None,
                      store_dtype: torch.dtype = torch.bfloat16, device="cpu") -> dict[str, torch.Tensor]:
    arch, cfg = load_config(raw_config)
    model = DecoderModel(arch.assemble(cfg))
    out: dict[str, torch.Tensor] = {}
    for e in model.expected_tensors():
        out[e.name] = random_tensor(seed, e.name, e.decl.shape, e.decl.role, std=std_of(e.name, std, std_overrides),
                                    gain_std=gain_std, device=device, dtype=store_dtype)
    return out


def write_random_model(raw_config: Mapping[str, Any], out_dir: str | os.PathLike, seed: int, *,
                       std: float = 0.02, gain_std: float = 0.1,
                       std_overrides: Mapping[str, float] | None = None,
                       store_dtype: torch.dtype = torch.bfloat16) -> str:
    """Write ``config.json`` and ``model.safetensors`` into ``out_dir``; return the folder."""
    out_dir = os.fspath(out_dir)
    os.makedirs(out_dir, exist_ok=True)
    state = random_state_dict(raw_config, seed, std=std, gain_std=gain_std,
                              std_overrides=std_overrides, store_dtype=store_dtype)
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(dict(raw_config), f, indent=1)
    write_safetensors(os.path.join(out_dir, "model.safetensors"), state,
                      metadata={"format": "pt", "seed": str(seed)})
    return out_dir
