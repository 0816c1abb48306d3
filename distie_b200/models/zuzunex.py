"""Recipe of the Zuzunex decoder: typed configuration -> parts and run order.

The design: layers in the order the configuration lists them, each a ``pre_norm`` block with layer norms (weight
and bias): ``x += mixer(norm_1(x))``, ``x += ff(norm_2(x))`` (a layer may have no feed-forward); a final layer norm;
an untied head whose logits are multiplied by a constant.  A stretch of layers may run several times in a row with
the same weights (``loop``): in the run order those layers are named once per pass, every pass with a cache slot (and
state slot) of its own.  Both mixers are grouped-query softmax attention with a learned sink per head in the
softmax's denominator and an output gate ``sigmoid(W_g h)`` on the concatenated heads:

* ``attention``: no rotation; q and k divided by their root mean square per head; q times a temperature that grows
  with the logarithm of the position; scores capped by ``cap * tanh(s / cap)``.
* ``attention_2``: q, k, v with biases, then a short causal convolution over time on every channel, then a weighted
  root-mean-square norm of q and k per head, then a rotation of the first ``dims`` elements of each head (halves
  paired) whose long waves are slowed along a ramp over the pair index, with a factor on cos and sin.

Feed-forwards: dense SwiGLU, or routed: softmax scores over all router outputs, the choice made on scores plus a
stored correction, the chosen scores renormalised as weights on the experts' outputs, the router's last outputs
standing for experts that return their input, and a shared expert for every token.

Tensor names: ``embed``; ``l<i>.norm1|norm2`` (+ ``.b``); ``l<i>.mix.q|k|v|g|o|sink`` and, for ``attention_2``,
``l<i>.mix.q.b|k.b|v.b``, ``l<i>.mix.q.conv|k.conv|v.conv``, ``l<i>.mix.q.norm|k.norm``; ``l<i>.mlp.gate|up|down``
(dense) or ``l<i>.mlp.router|correction``, ``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down``;
``final.norm`` (+ ``.b``); ``head``.
"""

from __future__ import annotations

import math

from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture
from ..config.zuzunex_config import DenseSizes, ZuzunexConfig

_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g", "sink": "sink"}


def _norm(eps: float, prefix: str, name: str) -> PartSpec:
    return PartSpec("layernorm", {"eps": eps, "weight": name, "bias": name + ".b"}, prefix)


def _mixer(m, prefix: str, eps: float) -> PartSpec:
    params = {"num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
              "scale": m.scale, "names": _NAMES, "bias_suffix": ".b", "qkv_bias": m.biases, "sink": True,
              "gate": "sigmoid", "norm_first": eps, "norm_weights": m.weighted_norm, "softcap": m.softcap,
              "q_temp": (m.temp_coef, m.temp_every) if m.temp_coef is not None else None, "conv": m.conv}
    if m.rot_dims:
        scaling = m.rot_scaling
        params["position"] = PartSpec("rotary", {
            "head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
            "factor": 0.1 * math.log(scaling.factor) + 1.0 if scaling is not None else 1.0,
            "scaling": ({"factor": scaling.factor, "original": scaling.original, "fast": scaling.fast, "slow": scaling.slow}
                        if scaling is not None else None)})
    return PartSpec("gqa_attention", params, prefix)


def _feed_forward(mlp, prefix: str) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    if isinstance(mlp, DenseSizes):
        return PartSpec("swiglu", {"intermediate_size": mlp.ff, "names": ("gate", "up", "down")}, prefix)
    return PartSpec(
        "routed_swiglu",
        {"experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "shared_size": mlp.shared_ff,
         "weight_on": "output", "scoring": "softmax", "correction": "correction", "normalise": True,
         "identity": mlp.identity},
        prefix,
    )


def zuzunex_recipe(cfg: ZuzunexConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norms = {"input": _norm(cfg.eps, p, "norm1")}
        if layer.mlp is not None:
            norms["post_mixer"] = _norm(cfg.eps, p, "norm2")
        layers.append(LayerSpec("pre_norm", _mixer(layer.mixer, p + "mix.", cfg.eps), _feed_forward(layer.mlp, p + "mlp."), norms))
    # A layer that runs again keeps its weights and gets a cache slot of its own for every pass.
    order = tuple(LayerCall(layer, slot, True) for slot, layer in enumerate(cfg.run_order()))
    return ModelSpec(
        architecture="Zuzunex",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        layers=tuple(layers),
        order=order,
        final_norm=_norm(cfg.eps, "final.", "norm"),
        embedding_name="embed",
        head_name="head",
        eos_token_id=cfg.eos_token_id,
        logit_scale=cfg.logit_scale if cfg.logit_scale != 1.0 else None,
        tolerated=tuple(f"l{i}.norm2{s}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for s in ("", ".b")),
    )


register_architecture("Zuzunex", ZuzunexConfig, zuzunex_recipe)
