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


def routed_ff(h, w, p, mlp):
    router, groups = mlp["router"], mlp["router"]["groups"]
    scores = torch.sigmoid((h @ w[p + "router"].T).to(torch.float32)).to(h.dtype)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in choose_experts(scores[t], int(router["top"]), int(groups["count"]), int(groups["keep"])):
            out[t] += float(router["scale"]) * scores[t, e] * capped_expert(h[t : t + 1], w, f"{p}e{e}.", float(mlp["expert"]["limit"]))[0]
    if mlp.get("shared") is not None:
        share = torch.sigmoid(h @ w[p + "shared.sg"].T)  # [T, 1]
        out = out + share * capped_expert(h, w, p + "shared.", float(mlp["shared"]["limit"]))
    return out


def feed_forward(h, w, p, mlp):
    if mlp["kind"] == "dense":
        return dense_ff(h, w, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, w, p, mlp)
    raise ValueError(mlp["kind"])


# -- the model -----------------------------------------------------------------------------------------------------
def forward(ids, w, cfg, dtype=torch.float64, layer_outputs=None):
    """Logits ``[T, vocab]`` of one sequence from its first token; ``layer_outputs`` (a list) receives the residual
    stream after every layer."""
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
            x = x + feed_forward(stored(rms_norm(x, w[p + "norm2"], eps)), w, p + "mlp.", layer["mlp"])
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    return stored(rms_norm(x, w["final.norm"], eps)) @ w["head"].T


def logit_scale(logits: torch.Tensor) -> float:
    centred = logits - logits.mean(-1, keepdim=True)
    return float(centred.pow(2).mean().sqrt())


_ = math  # (kept for callers that build configurations with it)
