"""Attention through a latent: keys and values of all heads are made from one small vector per token.

Per token, with ``h`` the mixer's input::

    c_q = rms_norm(W_dq h) * w_q                      query latent            [q_rank]
    q   = W_uq c_q                                    per head [dim plain | rot_dim to rotate]
    d   = W_dkv h                                     [kv_rank + rot_dim]
    c   = rms_norm(d[:kv_rank]) * w_kv                key/value latent        [kv_rank]
    r   = rotate(d[kv_rank:], position)               one rotated key part, shared by all heads
    key_h = [W_uk,h c | r],  value_h = W_uv,h c
    score_h(i, j) = (q_plain,h(i) . W_uk,h c(j) + rotate(q_rot,h(i)) . r(j)) * scale,   j <= i
    weights = exp(score) / (sum_j exp(score) + exp(sink_h))       (``sink``: one learned number per head)
    out = W_o concat_h(sigmoid((W_g h)_h) * sum_j weights_h(i, j) value_h(j))

Only ``[c | r]`` is cached, one row per token (a cache group of one kv head whose values are the first
``kv_rank`` columns of its keys).  Nothing is expanded per head when the cache is read: since
``q_plain . (W_uk c) = (W_uk^T q_plain) . c``, the plain part of a query is folded into the latent's space
(``kv_rank`` numbers per head), the attention mixes cached latents, and ``W_uv`` is applied to the mix.  A step
of one token and a portion of a prompt run the same ops.

A layer with ``own_latent=False`` has no ``W_dkv``: it reads the rows that the owner of its cache slot stored
(after that layer's norm and rotation), with its own ``W_uk``, ``W_uv``, queries, sink, gate and output.

The projections that read ``h`` (``W_dq``, ``W_dkv``, ``W_g``) are one product against the row-stacked weight;
both norms, the rotation of ``r`` and the store of the cache row are one op on its float32 accumulators.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, POSITION_ENCODINGS, BuildContext, CacheNeed, LayerRun, TensorSpec, build_part
from .linear import fuse_rows


@MIXERS.register("latent_attention")
class LatentAttention:
    """params: ``num_heads``, ``head_dim`` (plain query/key dimensions per head), ``rot_dim``, ``value_dim``,
    ``kv_rank``, ``q_rank``, ``scale``, ``eps`` (of the two latent norms), ``position`` (a PartSpec; its table
    rotates the ``rot_dim`` part), ``sink`` (bool), ``gate`` (None or ``"head_sigmoid"``), ``own_latent`` (bool),
    ``names`` (what the tensors' names add to the prefix).

    tensors: ``dq [q_rank, hidden]``, ``dq.norm [q_rank]``, ``uq [heads * (head_dim + rot_dim), q_rank]``,
    ``dkv [kv_rank + rot_dim, hidden]`` and ``dkv.norm [kv_rank]`` (with a latent of its own),
    ``uk [heads * head_dim, kv_rank]``, ``uv [heads * value_dim, kv_rank]``, ``sink [heads]``,
    ``g [heads, hidden]``, ``o [hidden, heads * value_dim]``."""

    _NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
              "uv": "uv", "sink": "sink", "g": "g", "o": "o"}

    def __init__(self, prm: dict, kernels, position, down, q_norm, kv_norm, up_q, up_keys, up_values, sink, out) -> None:
        self.kernels = kernels
        self.position = position
        self.num_heads = int(prm["num_heads"])
        self.head_dim = int(prm["head_dim"])
        self.rot_dim = int(prm["rot_dim"])
        self.value_dim = int(prm["value_dim"])
        self.kv_rank = int(prm["kv_rank"])
        self.q_rank = int(prm["q_rank"])
        self.scale = float(prm["scale"])
        self.eps = float(prm["eps"])
        self.own_latent = bool(prm.get("own_latent", True))
        self.gated = bool(prm.get("gate"))
        self.down, self.q_norm, self.kv_norm = down, q_norm, kv_norm
        self.up_q, self.up_keys, self.up_values = up_q, up_keys, up_values
        self.sink, self.out = sink, out

    @classmethod
    def _name(cls, spec: PartSpec, which: str) -> str:
        return spec.prefix + spec.params.get("names", cls._NAMES).get(which, cls._NAMES[which])

    @staticmethod
    def _check(prm) -> None:
        for key in ("num_heads", "head_dim", "value_dim", "kv_rank", "q_rank"):
            if int(prm[key]) < 1:
                raise ValueError(f"{key} must be >= 1, got {prm[key]}")
        if int(prm["rot_dim"]) < 0:
            raise ValueError(f"rot_dim must be >= 0, got {prm['rot_dim']}")
        if int(prm["kv_rank"]) + int(prm["rot_dim"]) > 1024:
            raise ValueError("kv_rank + rot_dim: the latent attention kernels take rows of up to 1024 elements")
        if prm.get("gate") not in (None, "head_sigmoid"):
            raise ValueError(f"gate {prm['gate']!r}: None or 'head_sigmoid'")

    # -- declarations -------------------------------------------------------
    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        cls._check(spec.params)
        prm = spec.params
        heads, dim, rot, vdim = int(prm["num_heads"]), int(prm["head_dim"]), int(prm["rot_dim"]), int(prm["value_dim"])
        rank, q_rank = int(prm["kv_rank"]), int(prm["q_rank"])
        specs = [
            TensorSpec(cls._name(spec, "dq"), (q_rank, hidden_size)),
            TensorSpec(cls._name(spec, "dq_norm"), (q_rank,), "norm"),
            TensorSpec(cls._name(spec, "uq"), (heads * (dim + rot), q_rank)),
        ]
        if prm.get("own_latent", True):
            specs += [TensorSpec(cls._name(spec, "dkv"), (rank + rot, hidden_size)),
                      TensorSpec(cls._name(spec, "dkv_norm"), (rank,), "norm")]
        specs += [TensorSpec(cls._name(spec, "uk"), (heads * dim, rank)), TensorSpec(cls._name(spec, "uv"), (heads * vdim, rank))]
        if prm.get("sink"):
            specs.append(TensorSpec(cls._name(spec, "sink"), (heads,), "bias"))
        if prm.get("gate"):
            specs.append(TensorSpec(cls._name(spec, "g"), (heads, hidden_size)))
        specs.append(TensorSpec(cls._name(spec, "o"), (hidden_size, heads * vdim)))
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed | None:
        prm = spec.params
        if not prm.get("own_latent", True):
            return None
        return CacheNeed(1, int(prm["kv_rank"]) + int(prm["rot_dim"]), value_dim=int(prm["kv_rank"]), values_in_keys=True)

    @classmethod
    def state_need(cls, spec: PartSpec):
        return None

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "LatentAttention":
        cls._check(spec.params)
        prm, w = spec.params, ctx.weights
        heads, dim, vdim, rank = int(prm["num_heads"]), int(prm["head_dim"]), int(prm["value_dim"]), int(prm["kv_rank"])
        own = bool(prm.get("own_latent", True))
        # Everything that reads the mixer's input, row-stacked: query latent, (key/value latent, key part), gates.
        stacked = [w.matrix(cls._name(spec, "dq"))]
        if own:
            stacked.append(w.matrix(cls._name(spec, "dkv")))
        if prm.get("gate"):
            stacked.append(w.matrix(cls._name(spec, "g")))
        position = build_part(POSITION_ENCODINGS, prm.get("position") or PartSpec("none"), ctx)
        up_keys = w.matrix(cls._name(spec, "uk")).reshape(heads, dim, rank).contiguous()              # [h, dim, rank]
        up_values = w.matrix(cls._name(spec, "uv")).reshape(heads, vdim, rank).transpose(1, 2).contiguous()  # [h, rank, vdim]
        return cls(
            dict(prm), ctx.kernels, position, fuse_rows(stacked),
            w.vector(cls._name(spec, "dq_norm")), w.vector(cls._name(spec, "dkv_norm")) if own else None,
            w.matrix(cls._name(spec, "uq")), up_keys, up_values,
            w.vector(cls._name(spec, "sink")) if prm.get("sink") else None, w.matrix(cls._name(spec, "o")),
        )

    # -- the step -----------------------------------------------------------
    def forward(self, x: torch.Tensor, run: LayerRun):
        if run.kv is None:
            raise RuntimeError("attention through a latent needs a cache slot")
        if run.writes_cache != self.own_latent:
            raise RuntimeError("a layer with a latent of its own owns its cache slot; one without reads another's")
        k = self.kernels
        tokens = x.shape[0]
        table = self.position.rotary_table()
        proj = k.linear_split(x, self.down)  # float32 [S, T, q_rank (+ kv_rank + rot_dim) (+ heads)]
        q_latent = torch.empty((tokens, self.q_rank), dtype=x.dtype, device=x.device)
        k.latent_kv_write(proj, run.step, run.kv if self.own_latent else None, table, self.q_rank, self.q_norm,
                          self.kv_rank, self.kv_norm, self.rot_dim, self.eps, q_latent)
        q = k.linear(q_latent, self.up_q, None, torch.float32)
        folded, rotated = k.latent_queries(q, self.up_keys, run.step, table, self.num_heads, self.head_dim, self.rot_dim)
        mixed = torch.empty((self.num_heads, tokens, self.kv_rank), dtype=x.dtype, device=x.device)
        k.latent_attention(folded, rotated, run.step, run.kv, self.num_heads, self.kv_rank, self.rot_dim, self.scale,
                           self.sink, mixed)
        gate = proj[..., proj.shape[-1] - self.num_heads :] if self.gated else None
        heads_out = k.latent_values(mixed, self.up_values, gate, self.num_heads, self.value_dim)
        return k.linear_split(heads_out, self.out)  # summed by the norm that follows
