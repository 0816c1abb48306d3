"""A plain, slow Zuzunex decoder: one function per mechanism, whole sequences, no cache.

Written from the design's equations only; it shares no code with the engine.  A sequence is run
from its first token, so it is the oracle for every way of cutting and batching.

Notation: ``h`` is a sublayer's input ``[T, width]``; weights are ``[out, in]`` and applied as
``h @ W.T``; ``w`` maps a tensor name to its tensor; ``cfg`` is the dictionary of ``config.json``;
``p`` is a tensor-name prefix (``"l3.mix."``); ``m`` a mixer's or feed-forward's entry of ``cfg``.
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


# -- norms ---------------------------------------------------------------------------------------------------------
def layer_norm(x, weight, bias, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight + bias


def rms_unit(x, eps):
    """``x / sqrt(mean(x^2) + eps)`` over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


# -- what positions do ---------------------------------------------------------------------------------------------
def query_temperature(positions, coef, every, dtype):
    """``1 + coef * ln(floor((p + 1) / every) + 1)`` per position."""
    steps = torch.div(positions + 1, every, rounding_mode="floor").to(dtype)
    return 1.0 + coef * torch.log(steps + 1.0)


def yarn_frequencies(base, dims, scaling, dtype=torch.float64):
    """Frequencies of the ``dims / 2`` pairs and the factor on cos and sin.  With ``scaling`` (``factor``,
    ``original``, ``fast``, ``slow``) the pairs that turn fewer than ``slow`` times over ``original`` positions
    are slowed by ``factor``, the ones that turn more than ``fast`` times stay, a ramp over the pair index between."""
    i = torch.arange(dims // 2, dtype=dtype)
    freq = base ** (-2.0 * i / dims)
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, freq, mult, dims):
    """``x [T, heads, n]``: of the first ``dims`` dimensions, i and i + dims/2 turn by ``position * freq[i]``;
    cos and sin are both multiplied by ``mult``."""
    half = dims // 2
    angles = positions.to(x.dtype)[:, None] * freq.to(x.dtype)[None, :]
    cos, sin = (angles.cos() * mult)[:, None, :], (angles.sin() * mult)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def causal_conv(u, taps_weight):
    """``u [T, C]``, ``taps_weight [C, taps]``: ``y_t = sum_j w[:, j] * u_(t - taps + 1 + j)``, zeros before the start."""
    tokens, taps = u.shape[0], taps_weight.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=u.dtype), u], 0)
    out = torch.zeros_like(u)
    for j in range(taps):
        out += padded[j: j + tokens] * taps_weight[:, j]
    return out


# -- softmax over the past, with a cap on the scores and one more term in the denominator --------------------------
def sink_attention(q, k, v, scale, sink, softcap=None):
    """``q [T, H, n]``, ``k [T, G, n]``, ``v [T, G, m]``, ``sink [H]`` -> ``[T, H, m]``.  Head a reads key/value
    head ``a // (H / G)``; token i sees j <= i; ``s = q . k * scale``, then ``cap * tanh(s / cap)``; the weights are
    ``exp(s_ij) / (sum_j exp(s_ij) + exp(sink_a))``."""
    tokens, heads, _ = q.shape
    per = heads // k.shape[1]
    out = torch.zeros(tokens, heads, v.shape[2], dtype=q.dtype)
    for head in range(heads):
        scores = (q[:, head] @ k[:, head // per].T) * scale
        if softcap:
            scores = softcap * torch.tanh(scores / softcap)
        for i in range(tokens):
            s = scores[i, : i + 1]
            top = torch.maximum(s.max(), sink[head])
            e = torch.exp(s - top)
            out[i, head] = (e / (e.sum() + torch.exp(sink[head] - top))) @ v[: i + 1, head // per]
    return out


# -- the two mixers ------------------------------------------------------------------------------------------------
def attention_mixer(h, w, p, m, eps, positions):
    """No rotation; q and k unit-normed per head; a temperature on q that grows with the position; capped scores."""
    tokens = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(tokens, heads, dim)
    k = (h @ w[p + "k"].T).view(tokens, kv_heads, dim)
    v = (h @ w[p + "v"].T).view(tokens, kv_heads, vdim)
    q, k = rms_unit(q, eps), rms_unit(k, eps)
    temp = m.get("q_temp")
    if temp:
        q = q * query_temperature(positions, temp["coef"], temp["every"], h.dtype)[:, None, None]
    mixed = sink_attention(stored(q), stored(k), stored(v), m["scale"], w[p + "sink"], m.get("softcap"))
    gated = mixed.reshape(tokens, heads * vdim) * torch.sigmoid(h @ w[p + "g"].T)
    return stored(gated) @ w[p + "o"].T


def conv_attention_mixer(h, w, p, m, eps, positions):
    """Biased projections -> short causal convolution -> weighted norm of q and k -> partial rotation -> attention."""
    tokens = h.shape[0]
    heads, kv_heads, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    parts = {}
    for name in "qkv":
        u = h @ w[p + name].T + w[p + name + ".b"]
        parts[name] = causal_conv(u, w[p + name + ".conv"]) if m.get("conv") else u
    q = rms_unit(parts["q"].view(tokens, heads, dim), eps) * w[p + "q.norm"]
    k = rms_unit(parts["k"].view(tokens, kv_heads, dim), eps) * w[p + "k.norm"]
    v = parts["v"].view(tokens, kv_heads, vdim)
    rot = m.get("rot")
    if rot:
        freq, mult = yarn_frequencies(rot["base"], rot["dims"], rot.get("scaling"), h.dtype)
        q = rotate_half(q, positions, freq, mult, rot["dims"])
        k = rotate_half(k, positions, freq, mult, rot["dims"])
    mixed = sink_attention(stored(q), stored(k), stored(v), m["scale"], w[p + "sink"])
    gated = mixed.reshape(tokens, heads * vdim) * torch.sigmoid(h @ w[p + "g"].T)
    return stored(gated) @ w[p + "o"].T


# -- feed-forwards -------------------------------------------------------------------------------------------------
def silu(z):
    return z * torch.sigmoid(z)


def gated_ff(h, w, p):
    return stored(silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def choose_experts(scores, correction, top):
    """Per token the ``top`` largest of ``scores + correction`` (ties to the lower index) -> ids ``[T, top]``."""
    choice = scores + correction
    order = sorted(range(choice.shape[-1]), key=lambda e: (-float(choice[e]), e)) if choice.dim() == 1 else None
    if order is not None:
        return order[:top]
    return [sorted(range(choice.shape[1]), key=lambda e: (-float(row[e]), e))[:top] for row in choice]


def choice_margin(scores, correction, top):
    """Per token the gap between the last chosen and the first not chosen choice score, as a share of the former's
    size (what rounding does to a score grows with the score)."""
    ranked = (scores + correction).sort(-1, descending=True).values
    if ranked.shape[-1] <= top:
        return torch.full(ranked.shape[:-1], float("inf"))
    return (ranked[..., top - 1] - ranked[..., top]) / ranked[..., top - 1].abs().clamp_min(1e-30)


def routed_ff(h, w, p, mlp, margins=None):
    """Softmax scores over all router outputs; the choice adds a correction, the weights do not and are divided by
    their sum; the last ``identity`` outputs stand for experts that return their input; a shared expert is added."""
    router = mlp["router"]
    experts, identity, top = router["experts"], router.get("identity", 0), router["top"]
    logits = h.to(torch.float64 if h.dtype == torch.float64 else torch.float32) @ w[p + "router"].to(h.dtype).T
    scores = torch.softmax(logits, -1)
    correction = w[p + "correction"].to(h.dtype)
    if margins is not None:
        margins.append(choice_margin(scores, correction, top))
    out = torch.zeros_like(h)
    for t, chosen in enumerate(choose_experts(scores, correction, top)):
        picked = scores[t, chosen]
        weights = picked / (picked.sum() + 1e-20)
        for weight, e in zip(weights, chosen):
            assert e < experts + identity
            if e >= experts:
                out[t] += weight * h[t]
            else:
                out[t] += weight * gated_ff(h[t: t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_ff(h, w, p + "shared.")
    return out


def feed_forward(h, w, p, mlp, margins=None):
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return gated_ff(h, w, p)
    if mlp["kind"] == "moe":
        return routed_ff(h, w, p, mlp, margins)
    raise ValueError(mlp["kind"])


# -- the model -----------------------------------------------------------------------------------------------------
def run_order(cfg) -> list[int]:
    """Layer indices in the order they run: layers ``start .. stop - 1`` ``times`` times in a row, the rest once."""
    count = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(count))
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    return list(range(start)) + list(range(start, stop)) * times + list(range(stop, count))


def forward(ids, w, cfg, dtype=torch.float64, layer_outputs=None, margins=None):
    """Logits ``[T, vocab]`` of one sequence from its first token."""
    w = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in w.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(ids.numel())
    eps = cfg["norm"]["eps"]
    x = w["embed"][ids]
    for index in run_order(cfg):
        layer, p = cfg["layers"][index], f"l{index}."
        h = stored(layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps))
        mixer = {"attention": attention_mixer, "attention_2": conv_attention_mixer}[layer["type"]]
        x = x + mixer(h, w, p + "mix.", layer["mixer"], eps, positions)
        if layer.get("mlp") is not None:
            h = stored(layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps))
            x = x + feed_forward(h, w, p + "mlp.", layer["mlp"], margins)
        if layer_outputs is not None:
            layer_outputs.append(x.clone())
    x = stored(layer_norm(x, w["final.norm"], w["final.norm.b"], eps))
    return (x @ w["head"].T) * cfg.get("logit_scale", 1.0)


def logit_scale(logits: torch.Tensor) -> float:
    """Root mean square of the logits with each row's mean taken off: the unit the tests' tolerances are in."""
    centred = logits - logits.mean(-1, keepdim=True)
    return float(centred.pow(2).mean().sqrt())


# -- tensors a configuration asks for, and random ones -------------------------------------------------------------
def tensor_shapes(cfg) -> dict:
    width, shapes = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}

    def gated(prefix, ff):
        shapes[prefix + "gate"], shapes[prefix + "up"], shapes[prefix + "down"] = (ff, width), (ff, width), (width, ff)

    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        for norm in ("norm1",) + (("norm2",) if layer.get("mlp") is not None else ()):
            shapes[p + norm] = shapes[p + norm + ".b"] = (width,)
        q_out, k_out, v_out = m["heads"] * m["dim"], m["kv_heads"] * m["dim"], m["kv_heads"] * m["vdim"]
        for name, rows in (("q", q_out), ("k", k_out), ("v", v_out)):
            shapes[f"{p}mix.{name}"] = (rows, width)
            if layer["type"] == "attention_2":
                shapes[f"{p}mix.{name}.b"] = (rows,)
                if m.get("conv"):
                    shapes[f"{p}mix.{name}.conv"] = (rows, m["conv"])
        if layer["type"] == "attention_2":
            shapes[p + "mix.q.norm"] = shapes[p + "mix.k.norm"] = (m["dim"],)
        shapes[p + "mix.sink"] = (m["heads"],)
        shapes[p + "mix.g"] = (m["heads"] * m["vdim"], width)
        shapes[p + "mix.o"] = (width, m["heads"] * m["vdim"])
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            gated(p + "mlp.", mlp["ff"])
        else:
            router = mlp["router"]
            for e in range(router["experts"]):
                gated(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
            outputs = router["experts"] + router.get("identity", 0)
            shapes[p + "mlp.router"], shapes[p + "mlp.correction"] = (outputs, width), (outputs,)
            if mlp.get("shared"):
                gated(p + "mlp.shared.", mlp["shared"]["ff"])
    shapes["final.norm"] = shapes["final.norm.b"] = (width,)
    shapes["head"] = (cfg["vocab"], width)
    return shapes


def random_weights(cfg, seed: int, router_gain: float = 4.0) -> dict:
    """float32 weights, rounded to bfloat16 values: matrices ``N(0, 1 / in)``, norm scales around 1, small biases,
    sinks and corrections of a size that matters, routers with a gain so that choices are seldom close."""
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.rsplit(".", 1)[-1]
        if name.endswith((".norm1", ".norm2", "final.norm", ".q.norm", ".k.norm")):
            t = 1.0 + 0.2 * torch.randn(shape, generator=gen)
        elif leaf == "b":
            t = 0.1 * torch.randn(shape, generator=gen)
        elif leaf == "sink":
            t = 1.5 * torch.randn(shape, generator=gen)
        elif leaf == "correction":
            t = 0.05 * torch.randn(shape, generator=gen)
        elif leaf == "conv":
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[1]) + 0.5 * (torch.arange(shape[1]) == shape[1] - 1)
        elif leaf == "router":
            t = router_gain * torch.randn(shape, generator=gen) / math.sqrt(shape[1])
        elif name == "embed":
            t = torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / math.sqrt(shape[-1])
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out
