"""Position encodings.  A mixer is given one as a parameter.

``rotary``: the reference's default RoPE (worker/src/inference/qwen2/model.py:93-117):
``inv_freq[j] = 1 / theta**(2j / d)`` computed in float32 exactly as there, angles
``pos * inv_freq`` and their cos/sin evaluated in float32 inside the fused kernel,
pairs ``(j, j + d/2)`` (rotate-half).  ``rotary_dim < head_dim``, interleaved pairs and
a factor on cos and sin are parameters for other layer kinds, and so is ``scaling``, which divides the
frequencies of long waves: with wavelength ``l = 2 pi / f``, ``f`` stays where ``l < original / high``, becomes
``f / factor`` where ``l > original / low``, and in between ``(1 - s) f / factor + s f`` with
``s = (original / l - low) / (high - low)``.  A ``scaling`` with the keys ``fast`` and ``slow`` instead of ``low`` and
``high`` blends over the pair index: with ``index(t) = d ln(original / (2 pi t)) / (2 ln theta)`` (the pair that turns
``t`` times over ``original`` positions), ``lo = max(floor(index(fast)), 0)``, ``hi = min(ceil(index(slow)), d - 1)``
and ``r_j = clamp((j - lo) / max(hi - lo, 0.001), 0, 1)`` the frequency of pair ``j`` is ``r_j f / factor + (1 - r_j) f``
(:func:`ramped_frequencies`); such encodings usually also put ``0.1 ln(factor) + 1`` on cos and sin (``factor`` of the
encoding, given by the recipe).  ``none`` rotates nothing.

An encoding that is no table of frequencies (learned or additive positions, a rotation
that depends on more than the position) returns ``None`` from ``rotary_table()`` and
offers ``apply(qkv, step, num_heads, num_kv_heads, head_dim)`` instead: the mixer finishes
its projection, hands ``qkv [T, (heads + 2 kv_heads) * head_dim]`` over to be changed in
place, and the fused kernel then only stores the keys and values.
"""

from __future__ import annotations

import math

import torch

from ..config.model_spec import PartSpec
from ..kernels.interface import RotaryTable
from .base import POSITION_ENCODINGS, BuildContext


# Layers with the same parameters share one table (and one tensor of frequencies): what a kernel set derives
# from a table and a step's positions is then made once per step, not once per layer.
_TABLES: dict[tuple, RotaryTable] = {}


def scaled_frequencies(theta: float, rotary_dim: int, factor: float, low: float, high: float, original: float) -> torch.Tensor:
    """Rotary frequencies ``theta**(-2j / d)`` with the long waves slowed down, made in float64 and stored as float32."""
    freq = theta ** (-torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)
    wavelength = 2.0 * math.pi / freq
    blend = ((original / wavelength - low) / (high - low)).clamp(0.0, 1.0)
    mixed = (1.0 - blend) * freq / factor + blend * freq
    out = torch.where(wavelength < original / high, freq, torch.where(wavelength > original / low, freq / factor, mixed))
    return out.to(torch.float32)


def ramped_frequencies(theta: float, rotary_dim: int, factor: float, original: float, fast: float, slow: float) -> torch.Tensor:
    """Rotary frequencies ``theta**(-2j / d)``, slowed by ``factor`` along a ramp over the pair index that starts at the
    pair turning ``fast`` times over ``original`` positions and ends at the one turning ``slow`` times; made in
    float64 and stored as float32."""
    j = torch.arange(0, rotary_dim // 2, dtype=torch.float64)
    freq = theta ** (-2.0 * j / rotary_dim)

    def index_of(turns: float) -> float:
        return rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))

    lo = max(math.floor(index_of(fast)), 0)
    hi = min(math.ceil(index_of(slow)), rotary_dim - 1)
    ramp = ((j - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return (freq / factor * ramp + freq * (1.0 - ramp)).to(torch.float32)


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding:
    """params: ``head_dim``, ``theta``, optional ``rotary_dim``, ``interleaved``, ``factor``, ``scaling``
    (a mapping with ``factor``, ``original`` and either ``low``, ``high`` or ``fast``, ``slow``)."""

    def __init__(self, table: RotaryTable) -> None:
        self._table = table

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "RotaryEncoding":
        head_dim = int(spec.params["head_dim"])
        rotary_dim = int(spec.params.get("rotary_dim") or head_dim)
        theta = float(spec.params["theta"])
        if rotary_dim % 2 or rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {rotary_dim} must be even and at most head_dim {head_dim}")
        scaling = spec.params.get("scaling")
        by_turns = bool(scaling) and "fast" in scaling
        names = ("factor", "original", "fast", "slow") if by_turns else ("factor", "low", "high", "original")
        scaled = tuple(float(scaling[n]) for n in names) + (by_turns,) if scaling else None
        key = (theta, rotary_dim, bool(spec.params.get("interleaved", False)), float(spec.params.get("factor", 1.0)),
               str(ctx.device), scaled)
        table = _TABLES.get(key)
        if table is None:
            if scaled is None:
                inv_freq = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
            elif by_turns:
                inv_freq = ramped_frequencies(theta, rotary_dim, *scaled[:4])
            else:
                inv_freq = scaled_frequencies(theta, rotary_dim, *scaled[:4])
            table = _TABLES[key] = RotaryTable(inv_freq.to(ctx.device), *key[1:4])
        return cls(table)

    def rotary_table(self) -> RotaryTable | None:
        return self._table


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding:
    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "NoPositionEncoding":
        return cls()

    def rotary_table(self) -> RotaryTable | None:
        return None
