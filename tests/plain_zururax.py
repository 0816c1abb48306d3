"""A plain, slow Zururax decoder: one function per mechanism, whole sequences, no cache.

Written from the design's equations only; it shares no code with the engine.  A sequence is run
from its first token, so it is the oracle for every way of cutting and batching.

Notation: ``h`` is a sublayer's input ``[T, width]``; weights are ``[out, in]`` and applied as
``h @ W.T``; ``w`` maps a tensor name to its tensor; ``cfg`` is the dictionary of ``config.json``.
"""

from __future__ import annotations

import math

import torch


STORED = None  # a torch dtype: what an engine of that type hands from one product to the next is rounded to it


def stored(x):
    """``x`` as a 16-bit engine stores it between two products; unchanged unless :func:`stored_as` is active."""
    return x if STORED is None else x.to(STORED).to(x.dtype)


class stored_as:
    """``with stored_as(torch.bfloat16): forward(...)``: the plain implementation with the roundings of a 16-bit
    engine (everything else stays in the precision of the call)."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global STORED
        self.before, STORED = STORED, self.dtype

    def __exit__(self, *exc):
        global STORED
        STORED = self.before


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


# -- rotary positions, neighbouring dimensions paired ------------------------------------------------------------
def rotate_pairs(x, positions, base, dims):
    """``x [T, ..., n]``: of the first ``dims`` dimensions, 2i and 2i + 1 turn by ``position * base**(-2i / dims)``."""
    i = torch.arange(dims // 2, dtype=x.dtype)
    angles = positions.to(x.dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]
    while angles.dim() < x.dim():
        angles = angles.unsqueeze(1)
    cos, sin = angles.cos(), angles.sin()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# -- softmax over the past with one more term in the denominator -------------------------------------------------
def sink_softmax_attention(q, k, v, scale, sink):
    """``q, k [T, heads, n]``, ``v [T, heads, m]``, ``sink [heads]`` -> ``[T, heads, m]``; token i sees j <= i, and
    the weights are ``exp(s_ij) / (sum_j exp(s_ij) + exp(sink))``."""
    tokens, heads, _ = q.shape
    out = torch.zeros(tokens, heads, v.shape[2], dtype=q.dtype)
    for head in range(heads):
        scores = (q[:, head] @ k[:, head].T) * scale
        for i in range(tokens):
            s = scores[i, : i + 1]
            top = torch.maximum(s.max(), sink[head])
            e = torch.exp(s - top)
            out[i, head] = (e / (e.sum() + torch.exp(sink[head] - top))) @ v[: i + 1, head]
    return out


# -- the mixer: attention through a latent -----------------------------------------------------------------------
def kv_latent(h, w, p, m, eps, positions):
    """What a layer with a down projection of its own leaves for itself and for layers that read it: the normed
    latent ``[T, kv_rank]`` and the one rotated key part ``[T, rot_dim]`` that all heads share."""
    rank, rot = m["kv_rank"], m["rot_dim"]
    down = h @ w[p + "dkv"].T
    latent = stored(rms_norm(down[:, :rank], w[p + "dkv.norm"], eps))
    shared = stored(rotate_pairs(down[:, rank : rank + rot], positions, float(m["rot"]["base"]), int(m["rot"]["dims"])))
    return latent, shared


def latent_attention(h, w, p, m, eps, positions, latent, shared):
    tokens = h.shape[0]
    heads, dim, rot, vdim = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q_latent = stored(rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps))
    q = (q_latent @ w[p + "uq"].T).reshape(tokens, heads, dim + rot)
    q_rot = rotate_pairs(q[..., dim:], positions, float(m["rot"]["base"]), int(m["rot"]["dims"]))
    q = stored(torch.cat([q[..., :dim], q_rot], dim=-1))
    k_plain = stored(latent @ w[p + "uk"].T).reshape(tokens, heads, dim)
    v = stored(latent @ w[p + "uv"].T).reshape(tokens, heads, vdim)
    k = torch.cat([k_plain, shared[:, None, :].expand(tokens, heads, rot)], dim=-1)
    mixed = sink_softmax_attention(q, k, v, float(m["scale"]), w[p + "sink"])
    gate = torch.sigmoid(h @ w[p + "g"].T)  # [T, heads]
    mixed = stored(mixed * gate[:, :, None])
    return mixed.reshape(tokens, heads * vdim) @ w[p + "o"].T


# -- feed-forwards -------------------------------------------------------------------------------------------------
def dense_ff(h, w, p):
    return stored(torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def capped_expert(h, w, p, limit):
    g = torch.clamp(h @ w[p + "gate"].T, max=limit)
    u = torch.clamp(h @ w[p + "up"].T, -limit, limit)
    return stored(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def choose_experts(scores, top, group_count, group_keep):
    """``scores [experts]`` -> the indices of the chosen experts, the largest first (ties to the lower index)."""
    experts = scores.shape[0]
    size = experts // group_count
    group_score = []
    for g in range(group_count):
        members = sorted((float(s) for s in scores[g * size : (g + 1) * size]), reverse=True)
        group_score.append(sum(members[:2]))
    kept = sorted(range(group_count), key=lambda g: (-group_score[g], g))[:group_keep]
    allowed = [e for e in range(experts) if e // size in kept]
    return sorted(allowed, key=lambda e: (-float(scores[e]), e))[:top]


def choice_margin(scores, top, group_count, group_keep):
    """How far the choice is from another one: the smallest gap, in scores, between what was taken last and what was
    left out first, among the groups and among the eligible experts (infinite when nothing was left out)."""
    experts = scores.shape[0]
    size = experts // group_count
    gaps = []
    group_score = [sum(sorted((float(s) for s in scores[g * size : (g + 1) * size]), reverse=True)[:2]) for g in range(group_count)]
    ranked = sorted(range(group_count), key=lambda g: (-group_score[g], g))
    if group_keep < group_count:
        gaps.append(group_score[ranked[group_keep - 1]] - group_score[ranked[group_keep]])
    allowed = sorted((float(scores[e]) for e in range(experts) if e // size in ranked[:group_keep]), reverse=True)
    if top < len(allowed):
        gaps.append(allowed[top - 1] - allowed[top])
    return min(gaps) if gaps else float("inf")


def routed_ff(h, w, p, mlp, margins=None):
    router, groups = mlp["router"], mlp["router"]["groups"]
    scores = torch.sigmoid((h @ w[p + "router"].T).to(torch.float32)).to(h.dtype)
    out = torch.zeros_like(h)
    if margins is not None:
        margins.append(torch.tensor([choice_margin(scores[t], int(router["top"]), int(groups["count"]), int(groups["keep"]))
                                     for t in range(h.shape[0])], dtype=torch.float64))
    for t in range(h.shape[0]):
        for e in choose_experts(scores[t], int(router["top"]), int(groups["count"]), int(groups["keep"])):
            out[t] += float(router["scale"]) * scores[t, e] * capped_expert(h[t : t + 1], w, f"{p}e{e}.", float(mlp["expert"]["limit"]))[0]
    if mlp.get("shared") is not None:
        share = torch.sigmoid(h @ w[p + "shared.sg"].T)  # [T, 1]
        out = out + share * capped_expert(h, w, p + "shared.", float(mlp["shared"]["limit"]))
    return out


def feed_forward(h, w, p, mlp, margins=None):
    if mlp["kind"] == "dense":
        return dense_ff(h, w, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, w, p, mlp, margins)
    raise ValueError(mlp["kind"])


# -- the model -----------------------------------------------------------------------------------------------------
def forward(ids, w, cfg, dtype=torch.float64, layer_outputs=None, margins=None):
    """Logits ``[T, vocab]`` of one sequence from its first token; ``layer_outputs`` (a list) receives the residual
    stream after every layer, ``margins`` (a list) every router's :func:`choice_margin` per token."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    positions = torch.arange(len(ids))
    x = w["embed"][torch.as_tensor(ids, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    held = {}  # layer -> (latent, shared rotated key part)
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        p, m = f"l{i}.", layer["mixer"]
        h = stored(rms_norm(x, w[p + "norm1"], eps))
        if m.get("kv_from") is None:
            held[i] = kv_latent(h, w, p + "mix.", m, eps, positions)
        latent, shared = held[i if m.get("kv_from") is None else int(m["kv_from"])]
        x = x + latent_attention(h, w, p + "mix.", m, eps, positions, latent, shared)
        if layer.get("mlp") is not None:
            x = x + feed_forward(stored(rms_norm(x, w[p + "norm2"], eps)), w, p + "mlp.", layer["mlp"], margins)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return stored(rms_norm(x, w["final.norm"], eps)) @ w["head"].T


def logit_scale(logits: torch.Tensor) -> float:
    centred = logits - logits.mean(-1, keepdim=True)
    return float(centred.pow(2).mean().sqrt())


# -- the checkpoint of a configuration -----------------------------------------------------------------------------
def tensor_shapes(cfg) -> dict:
    width, shapes = cfg["width"], {"embed": (cfg["vocab"], cfg["width"]), "final.norm": (cfg["width"],), "head": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        heads, dim, rot, vdim, rank, q_rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        shapes[p + "norm1"] = (width,)
        shapes.update({p + "mix.dq": (q_rank, width), p + "mix.dq.norm": (q_rank,), p + "mix.uq": (heads * (dim + rot), q_rank),
                       p + "mix.uk": (heads * dim, rank), p + "mix.uv": (heads * vdim, rank), p + "mix.sink": (heads,),
                       p + "mix.g": (heads, width), p + "mix.o": (width, heads * vdim)})
        if m.get("kv_from") is None:
            shapes.update({p + "mix.dkv": (rank + rot, width), p + "mix.dkv.norm": (rank,)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = (width,)
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.up": (mlp["ff"], width), p + "mlp.down": (width, mlp["ff"])})
            continue
        shapes[p + "mlp.router"] = (mlp["router"]["experts"], width)
        for e in range(mlp["router"]["experts"]):
            ff = mlp["expert"]["ff"]
            shapes.update({f"{p}mlp.e{e}.gate": (ff, width), f"{p}mlp.e{e}.up": (ff, width), f"{p}mlp.e{e}.down": (width, ff)})
        if mlp.get("shared") is not None:
            ff = mlp["shared"]["ff"]
            shapes.update({p + "mlp.shared.gate": (ff, width), p + "mlp.shared.up": (ff, width),
                           p + "mlp.shared.down": (width, ff), p + "mlp.shared.sg": (1, width)})
    return shapes


def random_weights(cfg, seed: int) -> dict:
    """Weights as a bfloat16 checkpoint holds them (float32 tensors of bfloat16 values): matrices around
    ``in ** -0.5`` (query and key maps larger, so that scores spread over several units and the softmax is not flat),
    norm scales around one, sinks of a few units either way, the embedding divided by the configuration's scale."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".sink"):
            t = 1.5 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / float(cfg["embedding"]["scale"])
        else:
            gain = 2.5 if name.endswith((".uq", ".uk", ".dkv")) else (2.0 if name.endswith((".router", ".sg", ".g")) else 1.0)
            t = torch.randn(shape, generator=g) * gain * shape[-1] ** -0.5
        out[name] = t.to(torch.bfloat16).float()
    return out
