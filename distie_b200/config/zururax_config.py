"""Typed configuration of the Zururax decoder, read from ``config.json`` keys.

``config.json`` gives ``vocab``, ``width``, ``norm.eps``, ``embedding.scale`` and ``layers``, a list in which
every entry names its ``type`` (``"latent_attention"``), the sizes and constants of its ``mixer`` (``heads``,
``dim``, ``rot_dim``, ``vdim``, ``kv_rank``, ``q_rank``, ``scale``, ``rot: {base, dims}`` and, for a layer that
reads another layer's latent, ``kv_from``) and its feed-forward ``mlp``: ``{"kind": "dense", "ff"}``,
``{"kind": "moe", "router": {"experts", "top", "scale", "groups": {"count", "keep"}}, "expert": {"ff", "limit"},
"shared": {"ff", "limit"} or null}``, or null for a layer without one.  Nothing has a default: a key that is
missing is an error that names it.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping

from .qwen2_config import ConfigError
from .zelasun_config import _count, _divides, _get, _number


@dataclass(frozen=True)
class LatentAttentionSizes:
    """Softmax attention whose keys and values are made from one latent per token."""

    heads: int
    dim: int        # plain (unrotated) query/key dimensions per head
    rot_dim: int    # rotated query/key dimensions per head; the key's are one vector shared by all heads
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    kv_from: int | None  # the layer whose latent and rotated key part this layer reads; None: its own

    @classmethod
    def read(cls, raw, where: str) -> "LatentAttentionSizes":
        rot = _get(raw, "rot", where)
        source = raw.get("kv_from") if isinstance(raw, Mapping) else None
        if source is not None and (isinstance(source, bool) or not isinstance(source, int) or source < 0):
            raise ConfigError(f"{where}kv_from must be a layer's index, got {source!r}")
        out = cls(_count(raw, "heads", where), _count(raw, "dim", where), _count(raw, "rot_dim", where),
                  _count(raw, "vdim", where), _count(raw, "kv_rank", where), _count(raw, "q_rank", where),
                  _number(raw, "scale", where), _number(rot, "base", where + "rot."), _count(rot, "dims", where + "rot."),
                  source)
        if out.rot_dims % 2 or out.rot_dims > out.rot_dim:
            raise ConfigError(f"{where}rot.dims ({out.rot_dims}) must be even and at most rot_dim ({out.rot_dim})")
        return out


@dataclass(frozen=True)
class DenseFeedForwardSizes:
    ff: int

    @classmethod
    def read(cls, raw, where: str) -> "DenseFeedForwardSizes":
        return cls(_count(raw, "ff", where))


@dataclass(frozen=True)
class GroupedRoutedSizes:
    """Experts in groups of neighbours; capped gated experts; a shared expert behind a gate of its own."""

    experts: int
    top: int
    weight_scale: float
    group_count: int
    group_keep: int
    ff: int
    limit: float
    shared_ff: int | None   # None: no shared expert
    shared_limit: float | None

    @classmethod
    def read(cls, raw, where: str) -> "GroupedRoutedSizes":
        router = _get(raw, "router", where)
        groups = _get(router, "groups", where + "router.")
        expert = _get(raw, "expert", where)
        shared = raw.get("shared")
        out = cls(_count(router, "experts", where + "router."), _count(router, "top", where + "router."),
                  _number(router, "scale", where + "router."), _count(groups, "count", where + "router.groups."),
                  _count(groups, "keep", where + "router.groups."), _count(expert, "ff", where + "expert."),
                  _number(expert, "limit", where + "expert."),
                  _count(shared, "ff", where + "shared.") if shared is not None else None,
                  _number(shared, "limit", where + "shared.") if shared is not None else None)
        _divides(out.group_count, out.experts, where + "router.experts / router.groups.count")
        if out.group_keep > out.group_count:
            raise ConfigError(f"{where}router.groups.keep ({out.group_keep}) exceeds count ({out.group_count})")
        if out.top > out.group_keep * (out.experts // out.group_count):
            raise ConfigError(f"{where}router.top ({out.top}) exceeds the experts of the kept groups")
        if out.limit <= 0 or (out.shared_limit is not None and out.shared_limit <= 0):
            raise ConfigError(f"{where}expert.limit and shared.limit must be positive")
        return out


def _read_mlp(raw, where: str):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind == "dense":
        return DenseFeedForwardSizes.read(raw, where)
    if kind == "moe":
        return GroupedRoutedSizes.read(raw, where)
    raise ConfigError(f"{where}kind {kind!r}: this design has 'dense' and 'moe' feed-forwards")


@dataclass(frozen=True)
class ZururaxLayer:
    type: str                 # "latent_attention"
    mixer: LatentAttentionSizes
    mlp: Any                  # DenseFeedForwardSizes | GroupedRoutedSizes | None


@dataclass(frozen=True)
class ZururaxConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    layers: tuple[ZururaxLayer, ...]
    eos_token_id: int | None = None
    architecture: str = "Zururax"
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "ZururaxConfig":
        listed = _get(raw, "layers", "")
        if not isinstance(listed, (list, tuple)) or not listed:
            raise ConfigError("layers must be a non-empty list")
        layers = []
        for index, entry in enumerate(listed):
            where = f"layers[{index}]."
            kind = _get(entry, "type", where)
            if kind != "latent_attention":
                raise ConfigError(f"{where}type {kind!r}: this design has 'latent_attention' layers")
            mixer = LatentAttentionSizes.read(_get(entry, "mixer", where), where + "mixer.")
            if mixer.kv_from is not None:
                if mixer.kv_from >= index:
                    raise ConfigError(f"{where}mixer.kv_from ({mixer.kv_from}) must name an earlier layer")
                source = layers[mixer.kv_from].mixer
                if source.kv_from is not None:
                    raise ConfigError(f"{where}mixer.kv_from names layer {mixer.kv_from}, which has no latent of its own")
                if (source.kv_rank, source.rot_dim, source.rot_base, source.rot_dims) != (
                        mixer.kv_rank, mixer.rot_dim, mixer.rot_base, mixer.rot_dims):
                    raise ConfigError(f"{where}mixer: kv_rank, rot_dim and rot must equal those of layer {mixer.kv_from}")
            layers.append(ZururaxLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + "mlp.")))
        eos = raw.get("eos_token_id")
        known = {"architecture", "architectures", "layers", "norm", "vocab", "width", "embedding", "eos_token_id"}
        return cls(
            vocab=_count(raw, "vocab", ""),
            width=_count(raw, "width", ""),
            eps=_number(_get(raw, "norm", ""), "eps", "norm."),
            embedding_scale=_number(_get(raw, "embedding", ""), "scale", "embedding."),
            layers=tuple(layers),
            eos_token_id=int(eos) if eos is not None else None,
            extra={k: v for k, v in raw.items() if k not in known},
        )
