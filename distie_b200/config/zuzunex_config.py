"""Typed configuration of the Zuzunex decoder, read from ``config.json`` keys.

``config.json`` gives ``vocab``, ``width``, ``norm.eps``, ``logit_scale``, an optional ``loop``
(``{"start", "stop", "times"}``: layers ``start .. stop - 1`` run ``times`` times in a row) and ``layers``, a
list in which every entry names its ``type`` (``"attention"`` or ``"attention_2"``), the sizes and constants of
its ``mixer`` and its feed-forward ``mlp``.

Mixer keys, both types: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``.  ``"attention"`` adds ``softcap``
(optional) and ``q_temp: {coef, every}`` (optional); ``"attention_2"`` adds ``conv`` (taps of the short
convolution; optional) and ``rot: {base, dims, scaling: {factor, original, fast, slow}}`` (``rot`` and
``scaling`` optional).  Feed-forwards: ``{"kind": "dense", "ff"}``, ``{"kind": "moe", "router": {"experts",
"top", "identity"}, "expert": {"ff"}, "shared": {"ff"} or null}``, or null for a layer without one.  A key that
the design needs and the file lacks is an error that names it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .qwen2_config import ConfigError
from .zelasun_config import _count, _get, _number


def _optional(raw, key: str):
    return raw.get(key) if isinstance(raw, Mapping) else None


@dataclass(frozen=True)
class FrequencyScaling:
    """Slows the long waves of a rotary encoding by ``factor`` (see ``parts/position.py``, scaling by turns)."""

    factor: float
    original: float
    fast: float
    slow: float

    @classmethod
    def read(cls, raw, where: str) -> "FrequencyScaling":
        out = cls(_number(raw, "factor", where), _number(raw, "original", where), _number(raw, "fast", where),
                  _number(raw, "slow", where))
        if out.factor <= 0 or out.original <= 0 or out.fast <= 0 or out.slow <= 0:
            raise ConfigError(f"{where}factor, original, fast and slow must be positive")
        return out


@dataclass(frozen=True)
class SinkAttentionSizes:
    """Grouped-query softmax attention with a learned sink per head and an output gate; what else a layer of
    either type does to q and k is in the optional fields."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None = None        # scores become cap * tanh(score / cap)
    temp_coef: float | None = None      # q times 1 + coef * ln(floor((p + 1) / every) + 1)
    temp_every: float | None = None     # a positive number, usually whole
    biases: bool = False                # q, k and v have biases
    weighted_norm: bool = False         # the norm of q and k has a weight (shared by the heads)
    conv: int | None = None             # taps of the causal convolution behind the projections
    rot_base: float | None = None
    rot_dims: int | None = None
    rot_scaling: FrequencyScaling | None = None

    @classmethod
    def read(cls, raw, where: str, kind: str) -> "SinkAttentionSizes":
        common = dict(heads=_count(raw, "heads", where), kv_heads=_count(raw, "kv_heads", where),
                      dim=_count(raw, "dim", where), vdim=_count(raw, "vdim", where), scale=_number(raw, "scale", where))
        if common["heads"] % common["kv_heads"]:
            raise ConfigError(f"{where}heads ({common['heads']}) is no multiple of kv_heads ({common['kv_heads']})")
        if kind == "attention":
            temp = _optional(raw, "q_temp")
            cap = _optional(raw, "softcap")
            if temp is not None and _number(temp, "every", where + "q_temp.") <= 0:
                raise ConfigError(f"{where}q_temp.every must be positive")
            if cap is not None and _number(raw, "softcap", where) <= 0:
                raise ConfigError(f"{where}softcap must be positive")
            return cls(**common, softcap=float(cap) if cap is not None else None,
                       temp_coef=_number(temp, "coef", where + "q_temp.") if temp is not None else None,
                       temp_every=_number(temp, "every", where + "q_temp.") if temp is not None else None)
        rot, taps = _optional(raw, "rot"), _optional(raw, "conv")
        scaling = _optional(rot, "scaling")
        out = cls(**common, biases=True, weighted_norm=True,
                  conv=_count(raw, "conv", where) if taps is not None else None,
                  rot_base=_number(rot, "base", where + "rot.") if rot is not None else None,
                  rot_dims=_count(rot, "dims", where + "rot.") if rot is not None else None,
                  rot_scaling=FrequencyScaling.read(scaling, where + "rot.scaling.") if scaling is not None else None)
        if out.rot_dims is not None and (out.rot_dims % 2 or out.rot_dims > out.dim):
            raise ConfigError(f"{where}rot.dims ({out.rot_dims}) must be even and at most dim ({out.dim})")
        return out


@dataclass(frozen=True)
class DenseSizes:
    ff: int


@dataclass(frozen=True)
class RoutedSizes:
    """Experts chosen by softmax scores plus a correction; the last ``identity`` router outputs return their input."""

    experts: int
    identity: int
    top: int
    ff: int
    shared_ff: int | None

    @classmethod
    def read(cls, raw, where: str) -> "RoutedSizes":
        router = _get(raw, "router", where)
        shared = _optional(raw, "shared")
        identity = _optional(router, "identity") or 0
        if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
            raise ConfigError(f"{where}router.identity must be a count, got {identity!r}")
        out = cls(_count(router, "experts", where + "router."), identity, _count(router, "top", where + "router."),
                  _count(_get(raw, "expert", where), "ff", where + "expert."),
                  _count(shared, "ff", where + "shared.") if shared is not None else None)
        if out.top > out.experts + out.identity:
            raise ConfigError(f"{where}router.top ({out.top}) exceeds the router's outputs ({out.experts + out.identity})")
        return out


def _read_mlp(raw, where: str):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind == "dense":
        return DenseSizes(_count(raw, "ff", where))
    if kind == "moe":
        return RoutedSizes.read(raw, where)
    raise ConfigError(f"{where}kind {kind!r}: this design has 'dense' and 'moe' feed-forwards")


@dataclass(frozen=True)
class ZuzunexLayer:
    type: str                 # "attention" | "attention_2"
    mixer: SinkAttentionSizes
    mlp: Any                  # DenseSizes | RoutedSizes | None


@dataclass(frozen=True)
class ZuzunexConfig:
    vocab: int
    width: int
    eps: float
    logit_scale: float
    layers: tuple[ZuzunexLayer, ...]
    loop: tuple[int, int, int] | None = None  # (start, stop, times)
    eos_token_id: int | None = None
    architecture: str = "Zuzunex"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    def run_order(self) -> list[int]:
        """Layer indices in the order they run."""
        count = len(self.layers)
        if self.loop is None:
            return list(range(count))
        start, stop, times = self.loop
        return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZuzunexConfig":
        listed = _get(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            kind = _get(entry, "type", where)
            if kind not in ("attention", "attention_2"):
                raise ConfigError(f"{where}type {kind!r}: this design has 'attention' and 'attention_2' layers")
            mixer = SinkAttentionSizes.read(_get(entry, "mixer", where), where + "mixer.", kind)
            layers.append(ZuzunexLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + "mlp.")))
        loop = raw.get("loop")
        if loop is not None:
            start, stop, times = (_get(loop, key, "loop.") for key in ("start", "stop", "times"))
            for value in (start, stop, times):
                if isinstance(value, bool) or not isinstance(value, int):
                    raise ConfigError(f"loop.start, loop.stop and loop.times are integers, got {loop!r}")
            if not 0 <= start <= stop <= len(layers) or times < 1:
                raise ConfigError(f"loop {loop!r}: 0 <= start <= stop <= {len(layers)} layers and times >= 1")
            loop = (start, stop, times)
        eos = raw.get("eos_token_id")
        scale = raw.get("logit_scale")
        known = {"architecture", "architectures", "layers", "norm", "vocab", "width", "loop", "logit_scale", "eos_token_id"}
        return cls(
            vocab=_count(raw, "vocab", ""),
            width=_count(raw, "width", ""),
            eps=_number(_get(raw, "norm", ""), "eps", "norm."),
            logit_scale=_number(raw, "logit_scale", "") if scale is not None else 1.0,
            layers=tuple(layers),
            loop=loop,
            eos_token_id=int(eos) if eos is not None else None,
            extra={k: v for k, v in raw.items() if k not in known},
        )
