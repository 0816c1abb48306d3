"""Plain tensor-op versions of every kernel, with the kernels' own signatures.

Two uses.  The ``-m gpu`` tests check each CUDA kernel against the function of the
same name here, at sizes the engine does not use.  And the CPU tests hand a
:class:`RefKernels` to the engine in place of the CUDA set, so that cache
bookkeeping, batching, scheduling and trace replay run end to end on a machine
without a GPU.  The product never imports this file.
"""

from __future__ import annotations

import torch

from distie_b200.kernels.interface import KernelSet, KvSlot, Normed, RotaryTable, StepTensors, Terms


def embed(ids, table):
    return table[ids.long()].float()


def add_rmsnorm(delta, residual, weight, eps, dtype, rows_index=None):
    """Returns (new residual, normed).  With rows_index only those rows are normed and the residual is unchanged."""
    if delta is not None and delta.dim() == 3:  # float32 slices of a split product
        delta = delta.float().sum(0)
    summed = residual if delta is None else residual + delta.float()
    source = summed if rows_index is None else summed[rows_index.long()]
    variance = (source * source).mean(dim=-1, keepdim=True)
    normed = (source * torch.rsqrt(variance + eps)).to(dtype)
    out = (weight.float() * normed.float()).to(dtype)
    return (summed if rows_index is None else residual), out


def swiglu(gate_up):
    inter = gate_up.shape[1] // 2
    g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    return (g / (1 + torch.exp(-g)) * u).to(gate_up.dtype)


def rotate(x, positions, rotary: RotaryTable | None):
    """x [T, heads, d] -> rotated, float32 arithmetic, stored back in x.dtype."""
    if rotary is None:
        return x.clone()
    rot = rotary.rotary_dim
    angles = positions.float()[:, None] * rotary.inv_freq.float()[None, :]
    factor = float(getattr(rotary, "factor", 1.0))
    cos, sin = angles.cos()[:, None, :] * factor, angles.sin()[:, None, :] * factor
    xf = x.float()
    out = xf.clone()
    if rotary.interleaved:
        a, b = xf[..., 0:rot:2], xf[..., 1:rot:2]
        out[..., 0:rot:2] = a * cos - b * sin
        out[..., 1:rot:2] = b * cos + a * sin
    else:
        a, b = xf[..., : rot // 2], xf[..., rot // 2 : rot]
        out[..., : rot // 2] = a * cos - b * sin
        out[..., rot // 2 : rot] = b * cos + a * sin
    return out.to(x.dtype)


def rope_kv_write(qkv, step: StepTensors, kv: KvSlot | None, rotary, num_heads, num_kv_heads, head_dim,
                  bias=None, q_out=None):
    if qkv.dim() == 3:  # float32 slices of the projection: sum, add the bias, then as below on a copy
        dense = qkv.float().sum(0)
        if bias is not None:
            dense = dense + bias.float()
        dense = dense.to(q_out.dtype)
        rope_kv_write(dense, step, kv, rotary, num_heads, num_kv_heads, head_dim)
        q_out.copy_(dense[:, : num_heads * head_dim])
        return
    tokens = step.num_tokens
    q_end, k_end = num_heads * head_dim, (num_heads + num_kv_heads) * head_dim
    positions = step.positions[:tokens]
    q = rotate(qkv[:tokens, :q_end].reshape(tokens, num_heads, head_dim), positions, rotary)
    qkv[:tokens, :q_end] = q.reshape(tokens, q_end)
    if q_out is not None:
        q_out.copy_(qkv[:tokens, :q_end])
    if kv is None:
        return
    k = rotate(qkv[:tokens, q_end:k_end].reshape(tokens, num_kv_heads, head_dim), positions, rotary)
    v = qkv[:tokens, k_end:].reshape(tokens, num_kv_heads, head_dim)
    seats = step.seq_seat[step.token_seq[:tokens].long()].long()
    pos = positions.long()
    pages = kv.block_table[seats, pos // kv.page_size].long()
    if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
        raise IndexError("a new token's page is missing from its block table")
    kv.k[pages, :, pos % kv.page_size, :] = k
    kv.v[pages, :, pos % kv.page_size, :] = v


def attention(qkv, step: StepTensors, kv: KvSlot, num_heads, num_kv_heads, head_dim, window, scale, chunk=None,
              keep_first=0, softcap=0.0, sink=None):
    """Token by token: gather the visible keys of the token's request from its pages, softmax in float32."""
    tokens = step.num_tokens
    out = torch.zeros((tokens, num_heads * kv.v.shape[-1]), dtype=qkv.dtype, device=qkv.device)
    rep = num_heads // num_kv_heads
    for t in range(tokens):
        pos = int(step.positions[t])
        seat = int(step.seq_seat[int(step.token_seq[t])])
        first = max(0, pos - int(window) + 1) if window else 0
        if chunk:
            first = max(first, pos // int(chunk) * int(chunk))
        keys = torch.arange(first, pos + 1, device=qkv.device)
        if keep_first and first > 0:  # the request's first positions stay visible beside the window
            keys = torch.cat([torch.arange(0, min(int(keep_first), first), device=qkv.device), keys])
        pages = kv.block_table[seat, keys // kv.page_size].long()
        if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
            raise IndexError("a block table does not cover the keys a token attends to")
        k = kv.k[pages, :, keys % kv.page_size, :].float()  # [n, kv_heads, d]
        v = kv.v[pages, :, keys % kv.page_size, :].float()
        q = qkv[t, : num_heads * head_dim].reshape(num_heads, head_dim).float()
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        scores = torch.einsum("hd,nhd->hn", q, k) * scale
        if softcap and softcap > 0:
            scores = float(softcap) * torch.tanh(scores / float(softcap))
        if sink is not None:  # one more term in the denominator: a column that carries no value
            scores = torch.cat([scores, sink.float().reshape(num_heads, 1)], dim=-1)
        probs = torch.softmax(scores, dim=-1)[:, : keys.numel()]
        out[t] = torch.einsum("hn,nhd->hd", probs, v).reshape(-1).to(qkv.dtype)
    return out


def add_layernorm(delta, residual, weight, bias, eps, dtype, rows_index=None):
    """Returns (new residual, normed), like add_rmsnorm."""
    if isinstance(delta, Terms):
        delta = delta.total()
    elif delta is not None and delta.dim() == 3:
        delta = delta.float().sum(0)
    summed = residual if delta is None else residual + delta.float()
    source = summed if rows_index is None else summed[rows_index.long()]
    centred = source - source.mean(dim=-1, keepdim=True)
    variance = (centred * centred).mean(dim=-1, keepdim=True)
    out = (centred / torch.sqrt(variance + eps) * weight.float() + bias.float()).to(dtype)
    return (summed if rows_index is None else residual), out


def token_seats(step: StepTensors):
    return step.seq_seat[step.token_seq[: step.num_tokens].long()].long()


def kv_write(k, v, step: StepTensors, kv: KvSlot):
    tokens = step.num_tokens
    pos = step.positions[:tokens].long()
    pages = kv.block_table[token_seats(step), pos // kv.page_size].long()
    if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
        raise IndexError("a new token's page is missing from its block table")
    kv.k[pages, :, pos % kv.page_size, :] = k[:tokens].reshape(tokens, kv.k.shape[1], kv.k.shape[3]).to(kv.k.dtype)
    kv.v[pages, :, pos % kv.page_size, :] = v[:tokens].reshape(tokens, kv.v.shape[1], kv.v.shape[3]).to(kv.v.dtype)


def whole(x):
    """A float32 matrix, or the sum of the slices ``[S, T, n]`` it was handed over as."""
    return x.float().sum(0) if x.dim() == 3 else x.float()


def head_gate(x, logits, num_heads):
    tokens = x.shape[0]
    logits = whole(logits)
    gated = x.float().reshape(tokens, num_heads, -1) * torch.sigmoid(logits.float())[:, :, None]
    return gated.reshape(tokens, -1).to(x.dtype)


def _silu(z):
    return z * torch.sigmoid(z)


def _softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def short_conv(x, weight, bias, state, step: StepTensors, activation="silu", input_bias=None):
    """Token by token in the step's order: the request's window of inputs lives in ``state[seat]``."""
    tokens, taps = step.num_tokens, weight.shape[1]
    x = whole(x)
    if input_bias is not None:
        x = x + input_bias.float()
    seats = token_seats(step)
    out = torch.zeros((tokens, x.shape[1]), dtype=torch.float32, device=x.device)
    for t in range(tokens):
        seat = int(seats[t])
        current = x[t].float()
        acc = weight[:, taps - 1].float() * current
        for back in range(1, taps):
            acc = acc + weight[:, taps - 1 - back].float() * state[seat, taps - 1 - back]
        if taps > 1:
            state[seat] = torch.cat([state[seat, 1:], current[None]], dim=0)
        if bias is not None:
            acc = acc + bias.float()
        out[t] = _silu(acc) if activation == "silu" else acc
    return out


def linear_recurrence(rule, q, k, v, decay, write, state, step: StepTensors, heads, groups, key_dim, value_dim,
                      decay_rate=None, decay_bias=None, skip=None):
    tokens = step.num_tokens
    decay, write = whole(decay), whole(write)
    seats = token_seats(step)
    out = torch.zeros((tokens, heads * value_dim), dtype=torch.float32, device=q.device)
    rep = heads // groups
    for t in range(tokens):
        seat = int(seats[t])
        for head in range(heads):
            grp = head // rep
            qt = q[t, grp * key_dim : (grp + 1) * key_dim].float()
            kt = k[t, grp * key_dim : (grp + 1) * key_dim].float()
            vt = v[t, head * value_dim : (head + 1) * value_dim].float()
            s = state[seat, head]  # [value_dim, key_dim]
            if rule == "delta":
                qt = qt / torch.sqrt((qt * qt).sum() + 1e-6) * key_dim ** -0.5
                kt = kt / torch.sqrt((kt * kt).sum() + 1e-6)
                g = torch.exp(-torch.exp(decay_rate[head].float()) * _softplus(decay[t, head].float() + decay_bias[head].float()))
                s = g * s
                u = torch.sigmoid(write[t, head].float()) * (vt - s @ kt)
            else:
                dt = _softplus(write[t, head].float() + decay_bias[head].float())
                g = torch.exp(-torch.exp(decay_rate[head].float()) * dt)
                s = g * s
                u = dt * vt
            s = s + torch.outer(u, kt)
            state[seat, head] = s
            read = s @ qt
            if skip is not None:
                read = read + skip[head].float() * vt
            out[t, head * value_dim : (head + 1) * value_dim] = read
    return out


def gated_rmsnorm(x, gate, weight, eps, group, gate_first, dtype, activation="silu"):
    tokens, n = x.shape
    xf, gf = x.float(), (_silu(whole(gate)) if activation == "silu" else torch.sigmoid(whole(gate)))
    w = weight.float().repeat(n // weight.numel())
    if gate_first:
        xf = xf * gf
    parts = xf.reshape(tokens, n // group, group)
    normed = (parts / torch.sqrt((parts * parts).mean(-1, keepdim=True) + eps)).reshape(tokens, n) * w
    if not gate_first:
        normed = normed * gf
    return normed.to(dtype)


def flat_sum(value):
    """A pending value (None, a matrix, float32 slices or Terms) as one float32 matrix."""
    if value is None:
        return None
    if isinstance(value, Terms):
        return value.total()
    return value.float().sum(0) if value.dim() == 3 else value.float()


def norm_add_rmsnorm(delta, delta_weight, delta_eps, residual, weight, eps, dtype, rows_index=None):
    """Returns (new residual, normed)."""
    d = flat_sum(delta)
    if d is not None and delta_weight is not None:
        d = d * torch.rsqrt((d * d).mean(-1, keepdim=True) + delta_eps) * delta_weight.float()
    summed = residual if d is None else residual + d
    source = summed if rows_index is None else summed[rows_index.long()]
    out = (source * torch.rsqrt((source * source).mean(-1, keepdim=True) + eps) * weight.float()).to(dtype)
    return (summed if rows_index is None else residual), out


def qk_rope_norm_write(qk, bias, step: StepTensors, kv: KvSlot | None, rotary, num_heads, num_kv_heads, head_dim,
                       norm_eps, q_dtype):
    """Returns q [T, heads * head_dim]; stores k (rotated, normed) and v (the key as projected) in their pages."""
    tokens = step.num_tokens
    dense = whole(qk)[:tokens]
    if bias is not None:
        dense = dense + bias.float()
    positions = step.positions[:tokens]
    q = dense[:, : num_heads * head_dim].reshape(tokens, num_heads, head_dim)
    k = dense[:, num_heads * head_dim :].reshape(tokens, num_kv_heads, head_dim)
    v = k.clone()
    q, k = rotate(q, positions, rotary), rotate(k, positions, rotary)
    if norm_eps is not None:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + norm_eps)
        k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + norm_eps)
    if kv is not None:
        pos = positions.long()
        pages = kv.block_table[token_seats(step), pos // kv.page_size].long()
        if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
            raise IndexError("a new token's page is missing from its block table")
        kv.k[pages, :, pos % kv.page_size, :] = k.to(kv.k.dtype)
        kv.v[pages, :, pos % kv.page_size, :] = v.to(kv.v.dtype)
    return q.reshape(tokens, num_heads * head_dim).to(q_dtype)


def qkv_norm_write(qkv, bias, step: StepTensors, kv: KvSlot | None, rotary, num_heads, num_kv_heads, head_dim, value_dim,
                   norm_eps, q_weight, k_weight, q_temp, q_dtype):
    """Returns q [T, heads * head_dim]; stores k (normed, rotated) and v in their pages."""
    tokens = step.num_tokens
    q_end, k_end = num_heads * head_dim, (num_heads + num_kv_heads) * head_dim
    dense = whole(qkv)[:tokens, : k_end + num_kv_heads * value_dim]
    if bias is not None:
        dense = dense + bias.float()
    positions = step.positions[:tokens]
    q = dense[:, :q_end].reshape(tokens, num_heads, head_dim)
    k = dense[:, q_end:k_end].reshape(tokens, num_kv_heads, head_dim)
    v = dense[:, k_end:].reshape(tokens, num_kv_heads, value_dim)
    if norm_eps is not None:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + norm_eps)
        k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + norm_eps)
        if q_weight is not None:
            q = q * q_weight.float()
        if k_weight is not None:
            k = k * k_weight.float()
    q, k = rotate(q, positions, rotary), rotate(k, positions, rotary)
    if q_temp is not None:
        steps = torch.div((positions + 1).float(), float(q_temp[1]), rounding_mode="floor")
        q = q * (1.0 + float(q_temp[0]) * torch.log(steps + 1.0))[:, None, None]
    if kv is not None:
        pos = positions.long()
        pages = kv.block_table[token_seats(step), pos // kv.page_size].long()
        if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
            raise IndexError("a new token's page is missing from its block table")
        kv.k[pages, :, pos % kv.page_size, :] = k.to(kv.k.dtype)
        kv.v[pages, :, pos % kv.page_size, :] = v.to(kv.v.dtype)
    return q.reshape(tokens, q_end).to(q_dtype)


def activation(x, kind="silu", scale=1.0, scaled_columns=0):
    out = whole(x).clone()
    if kind == "silu":
        out = _silu(out)
    if scaled_columns:
        out[:, :scaled_columns] *= scale
    return out


def exp_gate_scan(log_in, log_forget, in_bias, forget_bias, cap, state, step: StepTensors):
    tokens = step.num_tokens
    i = cap * torch.tanh((whole(log_in)[:tokens] + in_bias.float()) / cap)
    f = torch.nn.functional.logsigmoid(cap * torch.tanh((whole(log_forget)[:tokens] + forget_bias.float()) / cap))
    seats = token_seats(step)
    keep, take, floor = torch.zeros_like(i), torch.zeros_like(i), torch.zeros_like(i)
    for t in range(tokens):
        seat = int(seats[t])
        before = state[seat].clone()
        now = torch.maximum(f[t] + before, i[t])
        keep[t], take[t], floor[t] = torch.exp(f[t] + before - now), torch.exp(i[t] - now), torch.exp(-now)
        state[seat] = now
    return keep, take, floor


def gated_recurrence(q, k, v, decay, write, state, step: StepTensors, heads, key_dim, value_dim, decay_rate, unit_column):
    tokens = step.num_tokens
    seats = token_seats(step)
    width = value_dim - 1 if unit_column else value_dim
    out = torch.zeros((tokens, heads * value_dim), dtype=torch.float32, device=q.device)
    decay = whole(decay) if decay is not None else None
    write = whole(write) if write is not None else None
    for t in range(tokens):
        seat = int(seats[t])
        for head in range(heads):
            qt = q[t, head * key_dim : (head + 1) * key_dim].float()
            kt = k[t, head * key_dim : (head + 1) * key_dim].float()
            vt = v[t, head * width : (head + 1) * width].float()
            if unit_column:
                vt = torch.cat([vt, torch.ones(1)])
            g = decay[t, head] if decay is not None else decay_rate[head].float()
            u = vt * write[t, head] if write is not None else vt
            s = g * state[seat, head] + torch.outer(u, kt)
            state[seat, head] = s
            out[t, head * value_dim : (head + 1) * value_dim] = s @ qt
    return out


def stabilized_readout(read, floor, heads, value_dim):
    tokens = read.shape[0]
    parts = read.float().reshape(tokens, heads, value_dim + 1)
    lower = torch.maximum(parts[:, :, value_dim].abs(), floor.float())
    return (parts[:, :, :value_dim] / (lower[:, :, None] + 1e-6)).reshape(tokens, heads * value_dim)


def glu(g, u, limit=None):
    """The hidden activation of a gated layer, float32: SwiGLU, or with a ``limit`` the capped form."""
    if limit is None:
        return _silu(g) * u
    g = torch.clamp(g, max=float(limit))
    u = torch.clamp(u, -float(limit), float(limit))
    return g * torch.sigmoid(1.702 * g) * (u + 1.0)


def route_top(x, router, top, scoring="sigmoid", groups=None, weight_scale=1.0, extra_rows=0, correction=None,
              normalise=False):
    logits = x.float() @ router.float().T
    experts = router.shape[0] - int(extra_rows)
    scores = torch.softmax(logits[:, :experts], -1) if scoring == "softmax" else torch.sigmoid(logits[:, :experts])
    if correction is not None or normalise:
        choice = scores + correction.float() if correction is not None else scores
        ids = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :top]
        weights = torch.gather(scores, 1, ids)
        if normalise:
            weights = weights / (weights.sum(-1, keepdim=True) + 1e-20)
        out = ids.to(torch.int32).contiguous(), (weights * float(weight_scale)).contiguous()
        return out if not extra_rows else (*out, logits[:, experts:].contiguous())
    allowed = scores.clone()
    if groups is not None and groups[0] > 1 and groups[1] < groups[0]:
        count, keep = int(groups[0]), int(groups[1])
        size = experts // count
        members = scores.reshape(-1, count, size)
        group_score = torch.sort(members, dim=-1, descending=True).values[..., :2].sum(-1)
        kept = torch.sort(group_score, dim=-1, descending=True, stable=True).indices[:, :keep]
        mask = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, kept, True)
        allowed = torch.where(mask[:, :, None].expand_as(members).reshape(-1, experts), scores, torch.full_like(scores, -1.0))
    weights, ids = torch.sort(allowed, dim=-1, descending=True, stable=True)
    out = ids[:, :top].to(torch.int32).contiguous(), (weights[:, :top] * float(weight_scale)).contiguous()
    return out if not extra_rows else (*out, logits[:, experts:].contiguous())


def routed_swiglu(x, ids, weights, gate_up, down, scale_input=True, limit=None, identity=0):
    tokens, top = ids.shape
    ff = gate_up.shape[1] // 2
    out = torch.zeros((top, tokens, x.shape[1]), dtype=torch.float32, device=x.device)
    for t in range(tokens):
        for j in range(top):
            e, w = int(ids[t, j]), weights[t, j].float()
            if gate_up.shape[0] <= e < gate_up.shape[0] + identity:  # an expert that returns its input
                out[j, t] = x[t].float() * w
                continue
            z = (x[t].float() * w).to(x.dtype).float() if scale_input else x[t].float()
            both = gate_up[e].float() @ z
            hidden = glu(both[:ff], both[ff:], limit).to(x.dtype).float()
            y = down[e].float() @ hidden
            out[j, t] = y if scale_input else y * w
    return out


def linear_glu(x, weight, dtype, limit=None, row_gate=None):
    both = x.float() @ weight.float().T
    ff = weight.shape[0] // 2
    hidden = glu(both[:, :ff], both[:, ff:], limit)
    if row_gate is not None:
        gate = whole(row_gate) if row_gate.dim() == 3 else row_gate.float()
        hidden = hidden * torch.sigmoid(gate.reshape(-1))[:, None]
    return hidden.to(dtype)


def linear_act(x, weight, dtype, kind="relu2"):
    z = x.float() @ weight.float().T
    if kind != "relu2":
        raise ValueError(kind)
    return (torch.relu(z) ** 2).to(dtype)


# -- attention through a latent ------------------------------------------------------------------------------------
def _unit_rms(x, weight, eps):
    return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * weight.float()


def latent_kv_write(proj, step: StepTensors, kv, rotary, q_rank, q_norm, kv_rank, kv_norm, rot_dim, eps, dtype):
    """Returns the normed query latent ``[T, q_rank]``; stores the token's row in ``kv.k`` (if ``kv``)."""
    tokens = step.num_tokens
    proj = whole(proj)[:tokens]
    q_latent = _unit_rms(proj[:, :q_rank], q_norm, eps).to(dtype)
    if kv is not None:
        latent = _unit_rms(proj[:, q_rank : q_rank + kv_rank], kv_norm, eps)
        part = proj[:, q_rank + kv_rank : q_rank + kv_rank + rot_dim]
        part = rotate(part[:, None, :], step.positions[:tokens], rotary)[:, 0]
        pos = step.positions[:tokens].long()
        pages = kv.block_table[token_seats(step), pos // kv.page_size].long()
        if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
            raise IndexError("a new token's page is missing from its block table")
        kv.k[pages, 0, pos % kv.page_size, :] = torch.cat([latent, part], dim=-1).to(kv.k.dtype)
    return q_latent


def latent_queries(q, up_keys, step: StepTensors, rotary, num_heads, dim, rot_dim, dtype):
    tokens = step.num_tokens
    q = whole(q)[:tokens].reshape(tokens, num_heads, dim + rot_dim)
    rotated = rotate(q[..., dim:], step.positions[:tokens], rotary).to(dtype)
    plain = q[..., :dim].to(dtype).float()
    folded = torch.einsum("thd,hdr->htr", plain, up_keys.float()).to(dtype)
    return folded.contiguous(), rotated.contiguous()


def latent_attention(folded, rotated, step: StepTensors, kv: KvSlot, num_heads, kv_rank, rot_dim, scale, sink):
    tokens = step.num_tokens
    out = torch.zeros((num_heads, tokens, kv_rank), dtype=folded.dtype, device=folded.device)
    for t in range(tokens):
        pos = int(step.positions[t])
        seat = int(step.seq_seat[int(step.token_seq[t])])
        keys = torch.arange(0, pos + 1, device=folded.device)
        pages = kv.block_table[seat, keys // kv.page_size].long()
        if bool(((pages < 0) | (pages >= kv.num_pages)).any()):
            raise IndexError("a block table does not cover the keys a token attends to")
        rows = kv.k[pages, 0, keys % kv.page_size, :].float()  # [n, kv_rank + rot_dim]
        scores = (folded[:, t].float() @ rows[:, :kv_rank].T + rotated[t].float() @ rows[:, kv_rank:].T) * scale  # [H, n]
        if sink is not None:
            scores = torch.cat([scores, sink.float()[:, None]], dim=1)
        probs = torch.softmax(scores, dim=-1)[:, : pos + 1]
        out[:, t] = (probs @ rows[:, :kv_rank]).to(folded.dtype)
    return out


def latent_values(mixed, up_values, gate, num_heads, value_dim, dtype):
    out = torch.einsum("htr,hrv->thv", mixed.float(), up_values.float())
    if gate is not None:
        out = out.to(dtype).float() * torch.sigmoid(whole(gate) if gate.dim() == 3 else gate.float())[:, :, None]
    return out.reshape(out.shape[0], num_heads * value_dim).to(dtype)


def sample(logits, temperatures, uniforms):
    picks = logits.float().argmax(dim=-1).to(torch.int32)
    if temperatures is None:
        return picks
    for row in range(logits.shape[0]):
        t = float(temperatures[row])
        if t > 0:
            z = logits[row].float() / t
            p = torch.exp(z - z.max())
            cdf = torch.cumsum(p.double(), dim=0)
            target = float(uniforms[row]) * float(cdf[-1])
            picks[row] = int(torch.searchsorted(cdf, torch.tensor(target, dtype=torch.float64), right=True).clamp(max=logits.shape[1] - 1))
    return picks


class RefKernels(KernelSet):
    """The interface of the CUDA kernel sets, computed with the functions above."""

    def __init__(self, dtype=torch.float32, device="cpu") -> None:
        self.dtype = dtype
        self.device = torch.device(device)
        self.launches = 0

    def embed(self, step, table, residual):
        residual[: step.num_tokens] = embed(step.token_ids[: step.num_tokens], table)

    def add_rmsnorm(self, delta, residual, weight, eps, out, rows_index=None):
        new_residual, normed = add_rmsnorm(delta, residual, weight, eps, self.dtype, rows_index)
        if rows_index is None and delta is not None:
            residual.copy_(new_residual)
        out.copy_(normed)

    def linear(self, x, weight, bias=None, out_dtype=None):
        y = torch.nn.functional.linear(x.float(), weight.float(), bias.float() if bias is not None else None)
        return y.to(out_dtype or self.dtype)

    def swiglu(self, gate_up, out):
        out.copy_(swiglu(gate_up))

    def rope_kv_write(self, qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias=None, q_out=None):
        rope_kv_write(qkv, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias, q_out)

    def attention(self, qkv, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale, chunk=None, keep_first=0,
                  softcap=0.0, sink=None):
        out.copy_(attention(qkv, step, kv, num_heads, num_kv_heads, head_dim, window, scale, chunk, keep_first, softcap, sink))

    def qkv_norm_write(self, qkv, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, value_dim, norm_eps,
                       q_weight, k_weight, q_temp, q_out):
        q_out.copy_(qkv_norm_write(qkv, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, value_dim, norm_eps,
                                   q_weight, k_weight, q_temp, q_out.dtype))

    def norm_add_rmsnorm(self, delta, delta_weight, delta_eps, residual, weight, eps, out, rows_index=None):
        new_residual, normed = norm_add_rmsnorm(delta, delta_weight, delta_eps, residual, weight, eps,
                                                out.dtype if out is not None else self.dtype, rows_index)
        if rows_index is None and delta is not None:
            residual.copy_(new_residual)
        if out is not None:
            out.copy_(normed)

    def qk_rope_norm_write(self, qk, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, norm_eps, q_out):
        q_out.copy_(qk_rope_norm_write(qk, bias, step, kv, rotary, num_heads, num_kv_heads, head_dim, norm_eps, q_out.dtype))

    def activation(self, x, kind="silu", scale=1.0, scaled_columns=0):
        return activation(x, kind, scale, scaled_columns)

    def exp_gate_scan(self, log_in, log_forget, in_bias, forget_bias, cap, state, step):
        return exp_gate_scan(log_in, log_forget, in_bias, forget_bias, cap, state, step)

    def stabilized_readout(self, read, floor, heads, value_dim):
        return stabilized_readout(read, floor, heads, value_dim)

    def route_top(self, x, router, top, scoring="sigmoid", groups=None, weight_scale=1.0, extra_rows=0, correction=None,
                  normalise=False):
        return route_top(x, router, top, scoring, groups, weight_scale, extra_rows, correction, normalise)

    def routed_swiglu(self, x, ids, weights, gate_up, down, scale_input=True, limit=None, identity=0):
        return routed_swiglu(x, ids, weights, gate_up, down, scale_input, limit, identity)

    def linear_glu(self, x, weight, limit=None, row_gate=None):
        return linear_glu(x, weight, self.dtype, limit, row_gate)

    def linear_act(self, x, weight, kind="relu2"):
        return linear_act(x, weight, self.dtype, kind)

    def latent_kv_write(self, proj, step, kv, rotary, q_rank, q_norm, kv_rank, kv_norm, rot_dim, eps, q_latent_out):
        q_latent_out.copy_(latent_kv_write(proj, step, kv, rotary, q_rank, q_norm, kv_rank, kv_norm, rot_dim, eps, self.dtype))

    def latent_queries(self, q, up_keys, step, rotary, num_heads, dim, rot_dim):
        return latent_queries(q, up_keys, step, rotary, num_heads, dim, rot_dim, self.dtype)

    def latent_attention(self, folded, rotated, step, kv, num_heads, kv_rank, rot_dim, scale, sink, out):
        out.copy_(latent_attention(folded, rotated, step, kv, num_heads, kv_rank, rot_dim, scale, sink))

    def latent_values(self, mixed, up_values, gate, num_heads, value_dim):
        return latent_values(mixed, up_values, gate, num_heads, value_dim, self.dtype)

    def add_layernorm(self, delta, residual, weight, bias, eps, out, rows_index=None):
        new_residual, normed = add_layernorm(delta, residual, weight, bias, eps, self.dtype, rows_index)
        if rows_index is None and delta is not None:
            residual.copy_(new_residual)
        out.copy_(normed)

    def kv_write(self, k, v, step, kv):
        kv_write(k, v, step, kv)

    def head_gate(self, x, logits, num_heads):
        x.copy_(head_gate(x, logits, num_heads))

    def short_conv(self, x, weight, bias, state, step, activation="silu", input_bias=None):
        return short_conv(x, weight, bias, state, step, activation, input_bias)

    def linear_recurrence(self, rule, q, k, v, decay, write, state, step, heads, groups, key_dim, value_dim,
                          decay_rate=None, decay_bias=None, skip=None, unit_column=False):
        if rule == "gated":
            return gated_recurrence(q, k, v, decay, write, state, step, heads, key_dim, value_dim, decay_rate, unit_column)
        return linear_recurrence(rule, q, k, v, decay, write, state, step, heads, groups, key_dim, value_dim,
                                 decay_rate, decay_bias, skip)

    def gated_rmsnorm(self, x, gate, weight, eps, group, gate_first, out, activation="silu"):
        out.copy_(gated_rmsnorm(x, gate, weight, eps, group, gate_first, out.dtype, activation))

    def sample(self, logits, temperatures, uniforms, out_tokens):
        out_tokens.copy_(sample(logits, temperatures, uniforms))

    def check_errors(self):
        return None
