"""Position encodings.  ``rotary``: tables of cos/sin(pos * f_i) with the llama3
frequency scaling, built in float64 and kept in float32
(crates/runner/src/llama31_engine.rs:115-168; the reference rounds its tables to
bfloat16, which this engine does not: angles and their functions stay 32-bit).
``none``: no position information is added (keys are stored as they are)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from .registry import BuildContext, register_position_encoding


def scaled_inverse_frequencies(rotary_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """f_i = theta^(-2i/d); llama3 scaling divides low frequencies by ``factor``, keeps
    high ones and blends in between (llama31_engine.rs:126-145).  float64."""
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    inv = 1.0 / (float(theta) ** (2.0 * i / rotary_dim))
    if not scaling:
        return inv
    if scaling.get("kind") == "yarn":
        return yarn_inverse_frequencies(rotary_dim, float(theta), scaling, inv)
    if scaling.get("kind") == "linear":           # every frequency divided by the factor (positions stretched)
        return inv / float(scaling["factor"])
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    old = float(scaling["original_max_position_embeddings"])
    wavelen = 2.0 * math.pi / inv
    smooth = (old / wavelen - low) / (high - low)
    blended = (1.0 - smooth) * inv / factor + smooth * inv
    return torch.where(wavelen > old / low, inv / factor,
                       torch.where(wavelen < old / high, inv, blended))


def yarn_inverse_frequencies(rotary_dim: int, theta: float, scaling: dict, inv: torch.Tensor) -> torch.Tensor:
    """Frequencies stretched by ``factor`` where a coordinate turns fewer than ``slow`` times over the
    ``original`` positions, kept where it turns more than ``fast`` times, blended linearly in between.

    The coordinate whose frequency makes n turns over the original length is
    c(n) = rotary_dim * ln(original / (2 pi n)) / (2 ln theta); with lo = max(floor(c(fast)), 0) and
    hi = min(ceil(c(slow)), rotary_dim - 1), coordinate i gets the share m_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
    of the stretched frequency: f_i / factor * m_i + f_i * (1 - m_i).  float64."""
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def coordinate(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(coordinate(float(scaling["fast"]))), 0)
    hi = min(math.ceil(coordinate(float(scaling["slow"]))), rotary_dim - 1)
    i = torch.arange(rotary_dim // 2, dtype=torch.float64)
    share = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return inv / factor * share + inv * (1.0 - share)


def table_gain(scaling: Optional[dict]) -> float:
    """What cos and sin are multiplied by: 0.1 ln(factor) + 1 under yarn scaling, else 1."""
    if scaling and scaling.get("kind") == "yarn":
        return 0.1 * math.log(float(scaling["factor"])) + 1.0
    return 1.0


@register_position_encoding("rotary")
class Rotary:
    """params: ``head_dim``, ``rotary_dim``, ``theta``, ``max_positions``, ``scaling`` (None, the llama3 keys,
    ``{"kind": "linear", "factor"}``, or ``{"kind": "yarn", "factor", "original", "fast", "slow"}``, which also
    scales the tables), ``pairing``
    (``"halves"``: coordinate i turns with i + rotary_dim/2, the default; ``"interleaved"``: 2i with 2i + 1).

    Interface of a position encoding: ``encode_and_append(ctx, qkv, kv, n_q, n_kv, write)``
    rotates the queries (and keys) of the packed ``qkv`` rows in place by each
    token's position and writes keys and values into the cache entry ``kv``.
    """

    def __init__(self, params, weights, build: BuildContext):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim", self.head_dim))
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and <= head_dim {self.head_dim}")
        pairing = params.get("pairing", "halves")
        if pairing not in ("halves", "interleaved"):
            raise ValueError(f"rotary pairing {pairing!r} is not known ('halves' or 'interleaved')")
        self.interleaved = pairing == "interleaved"
        n_pos = min(int(params["max_positions"]), int(build.max_positions))
        self.max_positions = n_pos
        inv = scaled_inverse_frequencies(self.rotary_dim, float(params["theta"]), params.get("scaling"))
        angle = torch.arange(n_pos, dtype=torch.float64, device=build.device)[:, None] \
            * inv.to(build.device)[None, :]
        gain = table_gain(params.get("scaling"))
        self.cos = (angle.cos() * gain).to(torch.float32).contiguous()
        self.sin = (angle.sin() * gain).to(torch.float32).contiguous()

    def check_range(self, batch) -> None:
        if batch.max_total > self.max_positions:
            raise ValueError(f"a sequence reaches {batch.max_total} tokens, beyond the "
                             f"{self.max_positions} positions this model encodes")

    def rotary_tables(self):
        """(cos, sin, rotary_dim) for kernels that rotate inside another operation."""
        return self.cos, self.sin, self.rotary_dim

    def encode_and_append(self, ctx, qkv, kv, n_q, n_kv, write_cache=True):
        self.check_range(ctx.batch)
        k_cache, v_cache, table, group = kv
        from ..cache import PAGE_SHIFT
        ctx.kernels.rope_append(qkv, self.cos, self.sin, ctx.batch, table, k_cache, v_cache, n_q, n_kv,
                                self.head_dim, self.rotary_dim, PAGE_SHIFT, write_cache, self.interleaved)


@register_position_encoding("none")
class NoPosition:
    def __init__(self, params, weights, build: BuildContext):
        self.head_dim = int(params["head_dim"])

    def encode_and_append(self, ctx, qkv, kv, n_q, n_kv, write_cache=True):
        k_cache, v_cache, table, group = kv
        from ..cache import PAGE_SHIFT
        ctx.kernels.rope_append(qkv, None, None, ctx.batch, table, k_cache, v_cache, n_q, n_kv,
                                self.head_dim, 0, PAGE_SHIFT, write_cache)
