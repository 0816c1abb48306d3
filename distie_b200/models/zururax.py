"""Recipe of the Zururax decoder: typed configuration -> parts and run order.

The design: token embeddings times a constant; layers in the order the configuration lists them, each a
``pre_norm`` block with RMS norms (``x += mixer(norm_1(x))``, ``x += ff(norm_2(x))``; a layer may have no
feed-forward); a final norm; an untied head.  Every mixer is an attention through a latent: queries and keys/values
are made from low-rank projections of the input, only the normed key/value latent and one rotated key part per
token are cached, the softmax has a learned sink per head and every head's output is gated by a sigmoid of a
projection of the layer's input.  A layer may read an earlier layer's cached rows instead of making its own
(``kv_from``): in the run order it is a call that writes no cache and names the other layer's slot.  Feed-forwards:
a dense one with the squared ReLU, or capped gated experts chosen by sigmoid scores among groups of experts, beside
a shared expert behind a gate of its own.

Tensor names: ``embed``; ``l<i>.norm1|norm2``; ``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|sink|g|o``;
``l<i>.mlp.up|down`` (dense) or ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down|sg``; ``final.norm``; ``head``.
"""

from __future__ import annotations

from ..config.model_spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.registry import register_architecture
from ..config.zururax_config import DenseFeedForwardSizes, ZururaxConfig


def _norm(eps: float, prefix: str, name: str) -> PartSpec:
    return PartSpec("rmsnorm", {"eps": eps, "name": name, "exact": True}, prefix)


def _mixer(m, prefix: str, eps: float) -> PartSpec:
    position = PartSpec("rotary", {"head_dim": m.rot_dim, "rotary_dim": m.rot_dims, "theta": m.rot_base,
                                   "interleaved": True})
    return PartSpec(
        "latent_attention",
        {"num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim, "kv_rank": m.kv_rank,
         "q_rank": m.q_rank, "scale": m.scale, "eps": eps, "position": position, "sink": True, "gate": "head_sigmoid",
         "own_latent": m.kv_from is None},
        prefix,
    )


def _feed_forward(mlp, prefix: str) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    if isinstance(mlp, DenseFeedForwardSizes):
        return PartSpec("activated", {"intermediate_size": mlp.ff, "activation": "relu2", "names": ("up", "down")}, prefix)
    return PartSpec(
        "routed_swiglu",
        {"experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "shared_size": mlp.shared_ff,
         "weight_on": "output", "weight_scale": mlp.weight_scale, "groups": (mlp.group_count, mlp.group_keep),
         "limit": mlp.limit, "shared_limit": mlp.shared_limit, "shared_gate": "sg" if mlp.shared_ff is not None else None},
        prefix,
    )


def zururax_recipe(cfg: ZururaxConfig) -> ModelSpec:
    layers, order, slot_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norms = {"input": _norm(cfg.eps, p, "norm1")}
        if layer.mlp is not None:
            norms["post_mixer"] = _norm(cfg.eps, p, "norm2")
        layers.append(LayerSpec("pre_norm", _mixer(layer.mixer, p + "mix.", cfg.eps), _feed_forward(layer.mlp, p + "mlp."), norms))
        if layer.mixer.kv_from is None:
            slot_of[i] = len(slot_of)
            order.append(LayerCall(i, slot_of[i], True))
        else:
            order.append(LayerCall(i, slot_of[layer.mixer.kv_from], False))
    return ModelSpec(
        architecture="Zururax",
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        layers=tuple(layers),
        order=tuple(order),
        final_norm=_norm(cfg.eps, "final.", "norm"),
        embedding_name="embed",
        head_name="head",
        eos_token_id=cfg.eos_token_id,
        embedding_scale=cfg.embedding_scale,
        # a layer without a feed-forward reads no second norm; a checkpoint may carry one all the same
        tolerated=tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.mlp is None),
    )


register_architecture("Zururax", ZururaxConfig, zururax_recipe)
