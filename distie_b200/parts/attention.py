"""Grouped-query attention over the paged cache.

Formulas of the reference (worker/src/inference/qwen2/model.py:138-225):
``q, k, v = x Wq^T + bq, ...``; rotation of q and k; the new k and v are stored
in their pages before anything is read (worker/src/inference/qwen2/paged_attn.py:
388-389); query head ``h`` reads kv head ``h // (heads / kv_heads)``; scores scaled
by ``head_dim**-0.5``; a token at position ``p`` sees keys ``<= p`` (and, with a
window ``w``, ``> p - w``); softmax in float32; output projection.

Beyond the reference: ``chunk`` (a token sees only the keys of its own chunk of that many
positions, counted from position 0 of the request), ``value_dim`` (values of another size than
keys), ``gate="head_sigmoid"`` (a projection ``g`` of the mixer's input to one number per head;
head h's output is multiplied by ``sigmoid(g_h)`` before the output projection) and ``names`` (what
the tensors are called in the checkpoint; ``bias_suffix`` what a bias adds to its matrix's name), ``values="keys"``
(no value projection: a token's value is its key as projected, bias included, before rotation and norm),
``qk_norm`` (an epsilon: after the rotation every head of q and k is divided by its root mean square) and
``keep_first`` (beside a window: the request's first positions stay visible to every later token).

A second family of options makes the layer run on the *prepared* path (one stacked projection ``[q | k | v | g]``
whose float32 accumulators are finished by one kernel before anything is rounded): ``sink`` (a learned number per
head, ``sink [heads]``: the softmax's denominator also holds ``exp(sink_h)``; no key, no value, not scaled, not
capped), ``softcap`` (``score <- cap * tanh(score / cap)`` after the scale), ``gate="sigmoid"`` (``g`` projects to
``heads * value_dim`` numbers and the concatenated heads are multiplied by ``sigmoid(g)`` element by element),
``norm_first`` (an epsilon: every head of q and k is divided by its root mean square BEFORE the rotation;
``norm_weights=True`` then multiplies by ``<q>.norm`` and ``<k>.norm``, ``[head_dim]`` each, shared by the heads),
``q_temp = (coef, every)`` (q at position p times ``1 + coef * ln(floor((p + 1) / every) + 1)``) and ``conv`` (taps of a
causal convolution over time on every channel of the projected q, k and v, bias included, before norm and rotation:
``y_t = sum_j w[:, j] u_(t - taps + 1 + j)``, tensors ``<q>.conv`` etc. ``[rows, taps]``; the request's last ``taps - 1``
projected rows are its state).

The three projections are one product against the row-stacked weight; rotation
and cache write are one kernel; attention reads q from the same buffer.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import MIXERS, POSITION_ENCODINGS, BuildContext, CacheNeed, LayerRun, StateNeed, TensorSpec, build_part
from .linear import Linear, fuse_rows


@MIXERS.register("gqa_attention")
class GqaAttention:
    """params: ``num_heads``, ``num_kv_heads``, ``head_dim``, ``qkv_bias``, ``out_bias``,
    ``window`` (None: full), ``chunk`` (None: none), ``value_dim`` (None: ``head_dim``), ``gate`` (None or
    ``"head_sigmoid"``), ``scale`` (None: ``head_dim**-0.5``), ``position`` (a PartSpec), ``names``, ``bias_suffix``,
    ``values`` (``"projected"`` or ``"keys"``), ``qk_norm`` (None or an epsilon), ``keep_first`` (0); and for the
    prepared path ``sink`` (bool), ``softcap``, ``gate="sigmoid"``, ``norm_first`` (an epsilon), ``norm_weights``
    (bool), ``q_temp`` (``(coef, every)``), ``conv`` (taps).

    tensors: ``q_proj``/``k_proj``/``v_proj``/``o_proj`` ``.weight`` (and ``.bias``), ``g_proj.weight`` with a
    gate; ``names`` maps ``q, k, v, o, g`` to other names (biases then add ``.bias`` to the stem).
    """

    _NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
              "g": "g_proj.weight", "sink": "sink"}
    _PREPARED = ("sink", "softcap", "norm_first", "q_temp", "conv")
    graph_safe = True

    def __init__(self, qkv: Linear, out: Linear, position, params: dict, kernels, gate: Linear | None = None,
                 extras: dict | None = None) -> None:
        self.qkv = qkv
        self.out = out
        self.gate = gate
        self.position = position
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.window = params.get("window")
        self.chunk = params.get("chunk")
        self.keep_first = int(params.get("keep_first") or 0)
        self.values_are_keys = params.get("values", "projected") == "keys"
        self.qk_norm = params.get("qk_norm")
        self.scale = float(params.get("scale") or self.head_dim**-0.5)
        self.kernels = kernels
        # the prepared path: what the stacked projection is finished with
        self.prepared = self._is_prepared(params)
        self.softcap = float(params.get("softcap") or 0.0)
        self.norm_first = params.get("norm_first")
        self.q_temp = tuple(params["q_temp"]) if params.get("q_temp") else None
        self.taps = int(params.get("conv") or 0)
        self.gate_kind = params.get("gate")
        extras = extras or {}
        self.sink = extras.get("sink")
        self.q_norm_weight, self.k_norm_weight = extras.get("q_norm"), extras.get("k_norm")
        self.conv_weight = extras.get("conv")

    @classmethod
    def _is_prepared(cls, params) -> bool:
        return any(params.get(key) for key in cls._PREPARED) or params.get("gate") == "sigmoid"

    @classmethod
    def _name(cls, spec: PartSpec, which: str, bias: bool = False) -> str:
        name = spec.prefix + spec.params.get("names", cls._NAMES).get(which, cls._NAMES[which])
        if not bias:
            return name
        return (name[: -len(".weight")] if name.endswith(".weight") else name) + spec.params.get("bias_suffix", ".bias")

    @classmethod
    def _stem(cls, spec: PartSpec, which: str) -> str:
        name = cls._name(spec, which)
        return name[: -len(".weight")] if name.endswith(".weight") else name

    # -- declarations -------------------------------------------------------
    @classmethod
    def _check(cls, params) -> None:
        heads, kv_heads, dim = int(params["num_heads"]), int(params["num_kv_heads"]), int(params["head_dim"])
        if heads < 1 or kv_heads < 1 or heads % kv_heads:
            raise ValueError(f"num_heads ({heads}) must be a positive multiple of num_kv_heads ({kv_heads})")
        vdim = int(params.get("value_dim") or dim)
        if dim < 1 or dim > 256 or vdim < 1 or vdim > 256:
            raise ValueError(f"head_dim {dim} / value_dim {vdim}: the attention kernels take 1 to 256")
        for key in ("window", "chunk"):
            if params.get(key) is not None and int(params[key]) < 1:
                raise ValueError(f"{key} must be >= 1, got {params[key]}")
        if params.get("gate") not in (None, "head_sigmoid", "sigmoid"):
            raise ValueError(f"gate {params['gate']!r}: None, 'head_sigmoid' or 'sigmoid'")
        if cls._is_prepared(params):
            if params.get("values", "projected") == "keys" or params.get("qk_norm") is not None:
                raise ValueError("sink, softcap, gate='sigmoid', norm_first, q_temp and conv go with projected values and no qk_norm")
            if params.get("norm_weights") and params.get("norm_first") is None:
                raise ValueError("norm_weights goes with norm_first")
            if params.get("softcap") is not None and float(params["softcap"]) <= 0:
                raise ValueError(f"softcap must be positive, got {params['softcap']}")
            if params.get("q_temp") and float(params["q_temp"][1]) <= 0:
                raise ValueError("q_temp = (coef, every) with every > 0")
            if params.get("conv") and not 1 <= int(params["conv"]) <= 16:
                raise ValueError("the short convolution takes 1 to 16 taps")
            if params.get("out_bias") or params.get("keep_first"):
                raise ValueError("out_bias and keep_first are not served on the prepared path")
        if params.get("values", "projected") not in ("projected", "keys"):
            raise ValueError(f"values {params['values']!r}: 'projected' or 'keys'")
        if params.get("values") == "keys" and vdim != dim:
            raise ValueError("values that are the keys have the keys' size")
        if params.get("qk_norm") is not None and params.get("values") != "keys":
            raise ValueError("qk_norm goes with values='keys' (the op that rotates, norms and stores in one pass)")
        if int(params.get("keep_first") or 0) < 0 or (params.get("keep_first") and not params.get("window")):
            raise ValueError("keep_first is a non-negative count and goes with a window")

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        cls._check(spec.params)
        prm = spec.params
        vdim = int(prm.get("value_dim") or prm["head_dim"])
        q_out = prm["num_heads"] * prm["head_dim"]
        kv_out = prm["num_kv_heads"] * prm["head_dim"]
        v_out = prm["num_kv_heads"] * vdim
        own_values = prm.get("values", "projected") != "keys"
        specs = [
            TensorSpec(cls._name(spec, "q"), (q_out, hidden_size)),
            TensorSpec(cls._name(spec, "k"), (kv_out, hidden_size)),
        ]
        if own_values:
            specs.append(TensorSpec(cls._name(spec, "v"), (v_out, hidden_size)))
        if prm.get("gate"):
            gate_rows = prm["num_heads"] * (vdim if prm["gate"] == "sigmoid" else 1)
            specs.append(TensorSpec(cls._name(spec, "g"), (gate_rows, hidden_size)))
        specs.append(TensorSpec(cls._name(spec, "o"), (hidden_size, prm["num_heads"] * vdim)))
        if prm.get("sink"):
            specs.append(TensorSpec(cls._name(spec, "sink"), (prm["num_heads"],), "bias"))
        if prm.get("norm_weights"):
            specs += [TensorSpec(cls._stem(spec, n) + ".norm", (prm["head_dim"],), "norm") for n in "qk"]
        if int(prm.get("conv") or 0) > 0:
            specs += [TensorSpec(cls._stem(spec, n) + ".conv", (rows, int(prm["conv"])), "bias")
                      for n, rows in (("q", q_out), ("k", kv_out), ("v", v_out))]
        if prm.get("qkv_bias", False):
            specs += [
                TensorSpec(cls._name(spec, "q", True), (q_out,), "bias"),
                TensorSpec(cls._name(spec, "k", True), (kv_out,), "bias"),
            ]
            if own_values:
                specs.append(TensorSpec(cls._name(spec, "v", True), (v_out,), "bias"))
        if prm.get("out_bias", False):
            specs.append(TensorSpec(cls._name(spec, "o", True), (hidden_size,), "bias"))
        return specs

    @classmethod
    def cache_need(cls, spec: PartSpec) -> CacheNeed:
        prm = spec.params
        vdim = int(prm.get("value_dim") or prm["head_dim"])
        return CacheNeed(int(prm["num_kv_heads"]), int(prm["head_dim"]), prm.get("window"), prm.get("chunk"),
                         vdim if vdim != int(prm["head_dim"]) else None, int(prm.get("keep_first") or 0))

    @classmethod
    def state_need(cls, spec: PartSpec):
        prm = spec.params
        taps = int(prm.get("conv") or 0)
        if taps <= 1:
            return None
        vdim = int(prm.get("value_dim") or prm["head_dim"])
        channels = (prm["num_heads"] + prm["num_kv_heads"]) * prm["head_dim"] + prm["num_kv_heads"] * vdim
        return StateNeed((taps - 1, channels), torch.float32)  # the request's last projected q, k and v rows

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "GqaAttention":
        cls._check(spec.params)
        prm, w = spec.params, ctx.weights
        if cls._is_prepared(prm):
            return cls._build_prepared(spec, ctx)
        stacked = "qkv" if prm.get("values", "projected") != "keys" else "qk"
        weight = fuse_rows([w.matrix(cls._name(spec, n)) for n in stacked])
        bias = fuse_rows([w.vector(cls._name(spec, n, True)) for n in stacked]) if prm.get("qkv_bias", False) else None
        out_bias = w.vector(cls._name(spec, "o", True)) if prm.get("out_bias", False) else None
        position = build_part(POSITION_ENCODINGS, prm.get("position") or PartSpec("none"), ctx)
        gate = Linear(w.matrix(cls._name(spec, "g")), None, ctx.kernels) if prm.get("gate") else None
        return cls(
            Linear(weight, bias, ctx.kernels),
            Linear(w.matrix(cls._name(spec, "o")), out_bias, ctx.kernels),
            position,
            dict(prm),
            ctx.kernels,
            gate,
        )

    @classmethod
    def _build_prepared(cls, spec: PartSpec, ctx: BuildContext) -> "GqaAttention":
        """q, k, v and the gate read the same input: their matrices are stacked into one product."""
        prm, w = spec.params, ctx.weights
        names = "qkvg" if prm.get("gate") else "qkv"
        weight = fuse_rows([w.matrix(cls._name(spec, n)) for n in names])
        bias = fuse_rows([w.vector(cls._name(spec, n, True)) for n in "qkv"]) if prm.get("qkv_bias", False) else None
        extras = {}
        if prm.get("sink"):
            extras["sink"] = w.vector(cls._name(spec, "sink"))
        if prm.get("norm_weights"):
            extras["q_norm"], extras["k_norm"] = (w.vector(cls._stem(spec, n) + ".norm") for n in "qk")
        if int(prm.get("conv") or 0) > 0:
            extras["conv"] = torch.cat([w.vector(cls._stem(spec, n) + ".conv") for n in "qkv"], dim=0).contiguous()
        position = build_part(POSITION_ENCODINGS, prm.get("position") or PartSpec("none"), ctx)
        if position.rotary_table() is None and hasattr(position, "apply"):
            raise ValueError("the prepared path takes a rotary table or no rotation")
        return cls(Linear(weight, bias, ctx.kernels), Linear(w.matrix(cls._name(spec, "o")), None, ctx.kernels),
                   position, dict(prm), ctx.kernels, None, extras)

    # -- the step -----------------------------------------------------------
    def _forward_prepared(self, x: torch.Tensor, run: LayerRun):
        """The stacked projection stays float32 (the product's accumulators, as slices when the product was split);
        the convolution moves the request's state on; one kernel adds the bias, norms, rotates, applies the
        query's temperature, stores k and v in their pages and hands q over; the attention caps the scores and
        counts the sink; the gate reads its columns of the same projection."""
        k = self.kernels
        tokens = x.shape[0]
        proj = k.linear_split(x, self.qkv.weight)
        q_end = self.num_heads * self.head_dim
        channels = q_end + self.num_kv_heads * (self.head_dim + self.value_dim)
        qkv, bias = proj[..., :channels], self.qkv.bias
        if self.taps > 0:
            qkv = k.short_conv(qkv, self.conv_weight, None, run.state if self.taps > 1 else None, run.step, "none",
                               input_bias=bias)
            bias = None
        q = torch.empty((tokens, q_end), dtype=x.dtype, device=x.device)
        k.qkv_norm_write(qkv, bias, run.step, run.kv if run.writes_cache else None, self.position.rotary_table(),
                         self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, self.norm_first,
                         self.q_norm_weight, self.k_norm_weight, self.q_temp, q)
        mixed = torch.empty((tokens, self.num_heads * self.value_dim), dtype=x.dtype, device=x.device)
        k.attention(q, mixed, run.step, run.kv, self.num_heads, self.num_kv_heads, self.head_dim, self.window,
                    self.scale, self.chunk, 0, self.softcap, self.sink)
        if self.gate_kind == "sigmoid":  # one logit per element: every column is a "head" of one element
            k.head_gate(mixed, proj[..., channels:], self.num_heads * self.value_dim)
        elif self.gate_kind == "head_sigmoid":
            k.head_gate(mixed, proj[..., channels:], self.num_heads)
        return k.linear_split(mixed, self.out.weight)  # summed by the norm that follows

    def forward(self, x: torch.Tensor, run: LayerRun) -> torch.Tensor:
        if run.kv is None:
            raise RuntimeError("attention needs a cache slot")
        if self.prepared:
            return self._forward_prepared(x, run)
        k = self.kernels
        mixed = torch.empty((x.shape[0], self.num_heads * self.value_dim), dtype=x.dtype, device=x.device)
        table = self.position.rotary_table()
        if self.values_are_keys:
            # One projection [q | k]; what follows it (bias, the key kept as the value, rotation, the norm of every
            # head, the stores into the pages and of q) is one op on the product's float32 accumulators.
            if table is None and hasattr(self.position, "apply"):
                raise RuntimeError("values that are the keys go with a rotary table or no rotation")
            q = torch.empty((x.shape[0], self.num_heads * self.head_dim), dtype=x.dtype, device=x.device)
            k.qk_rope_norm_write(k.linear_split(x, self.qkv.weight), self.qkv.bias, run.step,
                                 run.kv if run.writes_cache else None, table, self.num_heads, self.num_kv_heads,
                                 self.head_dim, self.qk_norm, q)
            k.attention(q, mixed, run.step, run.kv, self.num_heads, self.num_kv_heads, self.head_dim, self.window,
                        self.scale, self.chunk, self.keep_first)
        elif self.keep_first:
            raise RuntimeError("keep_first is served for values='keys' layers only")
        elif self.value_dim != self.head_dim:
            # Values of another size than keys: nothing of the fused kernels fits; the projection is finished,
            # keys and values go to their pages as they are (such layers rotate nothing) and the size-agnostic
            # attention reads q from the projection's first columns.
            if table is not None or hasattr(self.position, "apply"):
                raise RuntimeError("a value size that differs from the key size goes with no rotation only")
            qkv = k.linear(x, self.qkv.weight, self.qkv.bias)
            q_end = self.num_heads * self.head_dim
            k_end = q_end + self.num_kv_heads * self.head_dim
            if run.writes_cache:
                k.kv_write(qkv[:, q_end:k_end], qkv[:, k_end:], run.step, run.kv)
            k.attention(qkv, mixed, run.step, run.kv, self.num_heads, self.num_kv_heads, self.head_dim, self.window,
                        self.scale, self.chunk)
        elif table is None and hasattr(self.position, "apply"):
            # An encoding of its own: the projection is finished here, the encoding changes q and k in
            # place, and the fused kernel only stores k and v and copies q out.
            q = torch.empty_like(mixed)
            qkv = k.linear(x, self.qkv.weight, self.qkv.bias)
            self.position.apply(qkv, run.step, self.num_heads, self.num_kv_heads, self.head_dim)
            k.rope_kv_write(qkv, run.step, run.kv if run.writes_cache else None, None, self.num_heads,
                            self.num_kv_heads, self.head_dim, q_out=q)
            k.attention(q, mixed, run.step, run.kv, self.num_heads, self.num_kv_heads, self.head_dim, self.window,
                        self.scale, self.chunk)
        else:
            # The projection, the bias, the rotation of q and k, the store of k and v in their pages and the
            # attention over the pages as one op of the kernel set, which may merge kernels for some steps.
            k.qkv_attention(x, self.qkv.weight, self.qkv.bias, run.step, run.kv, run.writes_cache, table,
                            self.num_heads, self.num_kv_heads, self.head_dim, self.window, self.scale, mixed, self.chunk)
        if self.gate is not None:
            k.head_gate(mixed, k.linear_split(x, self.gate.weight), self.num_heads)
        if self.out.bias is not None:
            return self.out(mixed)
        return k.linear_split(mixed, self.out.weight)  # summed by the norm that follows
