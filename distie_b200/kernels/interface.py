"""The set of operations the parts are written against.

Parts never call a kernel by name; they are handed a :class:`KernelSet` when they
are built.  The engine has two of them, both in :mod:`distie_b200.kernels.device`:
the bfloat16 set that serving uses and the float32 set in which every product,
sum and exponential is a true 32-bit operation.  Tests pass a third, written with
plain tensor operations, to check each kernel against and to run the engine's
bookkeeping on a machine without a GPU; the product never falls back to it.

Shapes (``T`` tokens of this step, ``B`` requests of this step):

``StepTensors``   the step's metadata on the device, all int32
    token_ids [T], positions [T], token_seq [T] (batch row of each token),
    seq_seat [B] (seat = row of the block tables and of the state slots).
``KvSlot``        one cache slot of one group
    k  [pages, kv_heads, page_size, head_dim], v  [pages, kv_heads, page_size, value_dim];
    block_table [seats, width] int32.  In a group whose values lie inside its keys (attention through
    a latent) ``v`` is a view of the first ``value_dim`` columns of ``k``.

Which keys a token sees: all keys up to its own position (``first_visible``), the last
``window`` of them, or those of its own ``chunk`` (positions ``chunk * n .. chunk * (n + 1) - 1``);
beside a window, the request's first ``keep_first`` positions when a layer keeps them.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass, field

import torch


Q_TILE = 128  # tokens per tile of StepTensors.q_tiles


@dataclass
class StepTensors:
    token_ids: torch.Tensor
    positions: torch.Tensor
    token_seq: torch.Tensor
    seq_seat: torch.Tensor
    num_tokens: int
    num_seqs: int
    num_decode_tokens: int  # the first this-many tokens are single-token rows
    max_kv_len: int = 0  # bound on the keys any token sees; a captured step uses a fixed bound
    q_tiles: torch.Tensor | None = None  # [n, 2] int32: (first token, rows <= Q_TILE) of each tile of the
    num_q_tiles: int = 0                 # multi-token entries; a tile holds consecutive tokens of one request
    derived: dict = field(default_factory=dict)  # what a kernel set made of this step once and its layers share


@dataclass
class KvSlot:
    k: torch.Tensor
    v: torch.Tensor
    block_table: torch.Tensor
    page_size: int
    num_pages: int


def first_visible(position: int, window: int | None = None, chunk: int | None = None) -> int:
    """The oldest key the token at ``position`` sees (it sees every key from there to itself)."""
    first = 0
    if window:
        first = max(first, position - int(window) + 1)
    if chunk:
        first = max(first, position // int(chunk) * int(chunk))
    return first


@dataclass
class Terms:
    """A sum that is still to be done: ``sum_i scale_i * tensor_i``, each tensor ``[T, hidden]`` or float32
    slices ``[S, T, hidden]`` (see :meth:`KernelSet.linear_split`).  A block whose sublayers all read one norm
    hands its sublayers' outputs over like this, and the norm kernel that follows adds them to the residual."""

    items: list  # of (tensor, scale)

    @classmethod
    def of(cls, value, scale: float = 1.0) -> "Terms":
        if isinstance(value, Terms):
            return cls([(t, s * scale) for t, s in value.items])
        return cls([(value, float(scale))])

    def __add__(self, other: "Terms") -> "Terms":
        return Terms(self.items + Terms.of(other).items)

    def flat(self) -> list:
        """``(float32 [T, hidden] matrix, scale)`` pairs: every slice on its own."""
        out = []
        for tensor, scale in self.items:
            if tensor.dim() == 3:
                out += [(tensor[i], scale) for i in range(tensor.shape[0])]
            else:
                out.append((tensor if tensor.dtype == torch.float32 else tensor.float(), scale))
        return out

    def total(self) -> torch.Tensor:
        """The sum itself, float32 ``[T, hidden]``, in the order of the items."""
        total = None
        for tensor, scale in self.flat():
            part = tensor if scale == 1.0 else tensor * scale
            total = part if total is None else total + part
        return total


@dataclass
class Normed:
    """A sublayer's output that is normalised before it joins the residual: ``rms_norm(sum of terms) * weight``.

    ``value`` is what a mixer or feed-forward returns (a matrix, float32 slices or :class:`Terms`); ``weight`` is
    the float32 scale of the norm (an offset the checkpoint leaves out is already added) and ``eps`` its epsilon.
    The norm kernel that follows does the sum, this norm, the addition to the residual and its own norm in one pass."""

    value: object
    weight: torch.Tensor
    eps: float


@dataclass(frozen=True)
class RotaryTable:
    """What the fused rotation kernel needs of a rotary position encoding."""

    inv_freq: torch.Tensor  # [rotary_dim / 2] float32
    rotary_dim: int
    interleaved: bool = False
    factor: float = 1.0  # cos and sin are multiplied by it (the attention factor of scaled rotary encodings)


class KernelSet(ABC):
    dtype: torch.dtype
    device: torch.device

    @abstractmethod
    def embed(self, step: StepTensors, table: torch.Tensor, residual: torch.Tensor) -> None:
        """residual[t] = table[token_ids[t]] as float32."""

    @abstractmethod
    def add_rmsnorm(self, delta, residual, weight, eps: float, out, rows_index=None) -> None:
        """residual += delta (float32, kept), out = weight * cast(residual * rsqrt(mean sq + eps)).

        ``delta`` is ``[T, hidden]`` in the set's dtype, or ``[S, T, hidden]`` float32 slices as
        :meth:`linear_split` returns them, which are added up in the same kernel.
        """

    @abstractmethod
    def linear(self, x, weight, bias=None, out_dtype=None):
        """x @ weight.T (+ bias); weight is [out, in]."""

    def linear_split(self, x, weight):
        """``x @ weight.T`` as float32 slices ``[S, T, out]`` whose sum over ``S`` is the product.

        A set that splits the reduction of a skinny product over several thread blocks returns
        the slices as they are and leaves the sum to the consumer (``add_rmsnorm``,
        ``rope_kv_write``), which saves the product a round of synchronisation.  The default is
        one slice.
        """
        return self.linear(x, weight, None, torch.float32).unsqueeze(0)

    @abstractmethod
    def swiglu(self, gate_up, out) -> None:
        """out = silu(gate_up[:, :I]) * gate_up[:, I:]."""

    def linear_swiglu(self, x, weight):
        """silu(x Wg^T) * (x Wu^T) for weight = [Wg; Wu] stacked along the rows; sets may fuse it."""
        gate_up = self.linear(x, weight)
        out = torch.empty((x.shape[0], weight.shape[0] // 2), dtype=gate_up.dtype, device=x.device)
        self.swiglu(gate_up, out)
        return out

    @abstractmethod
    def rope_kv_write(self, qkv, step: StepTensors, kv: KvSlot | None, rotary: RotaryTable | None,
                      num_heads: int, num_kv_heads: int, head_dim: int, bias=None, q_out=None) -> None:
        """Rotate q and k, store k and v of the new tokens in their pages (if kv).

        ``qkv`` is ``[T, (heads + 2 kv_heads) * head_dim]`` in the set's dtype with q rotated in
        place, or float32 slices ``[S, T, ...]`` of the projection (see :meth:`linear_split`), in
        which case the slices are summed, ``bias`` is added and the rotated q is written to
        ``q_out [T, heads * head_dim]``.
        """

    def qkv_rope_write(self, x, weight, bias, step: StepTensors, kv: KvSlot | None, rotary: RotaryTable | None,
                       num_heads: int, num_kv_heads: int, head_dim: int, q_out) -> None:
        """The q/k/v projection with what follows it: ``x @ weight.T + bias``, q and k rotated, q to
        ``q_out`` and k and v into their pages (if kv).  The default is the two ops after one another;
        a set may do it in the product's epilogue."""
        slices = self.linear_split(x, weight)
        self.rope_kv_write(slices, step, kv, rotary, num_heads, num_kv_heads, head_dim, bias=bias, q_out=q_out)

    def qkv_attention(self, x, weight, bias, step: StepTensors, kv: KvSlot, writes_cache: bool,
                      rotary: RotaryTable | None, num_heads: int, num_kv_heads: int, head_dim: int,
                      window: int | None, scale: float, out, chunk: int | None = None) -> None:
        """From the mixer's input to the attention's output: the q/k/v projection, bias, rotation, the new
        keys and values into their pages (if ``writes_cache``) and attention over the pages into ``out``.
        The default is the ops after one another; a set may merge them for some steps."""
        q = torch.empty((x.shape[0], num_heads * head_dim), dtype=out.dtype, device=x.device)
        self.qkv_rope_write(x, weight, bias, step, kv if writes_cache else None, rotary, num_heads, num_kv_heads,
                            head_dim, q)
        self.attention(q, out, step, kv, num_heads, num_kv_heads, head_dim, window, scale, chunk)

    @abstractmethod
    def attention(self, qkv, out, step: StepTensors, kv: KvSlot, num_heads: int, num_kv_heads: int,
                  head_dim: int, window: int | None, scale: float, chunk: int | None = None,
                  keep_first: int = 0, softcap: float = 0.0, sink=None) -> None:
        """Causal attention of every token over its request's pages, optionally only over the last
        ``window`` keys or over the keys of the token's own ``chunk``.  With a window, ``keep_first`` keeps
        the request's first that-many positions visible to every later token, at their true positions.
        The size of a value is the last dimension of ``kv.v`` and may differ from ``head_dim``; ``out`` is
        ``[T, heads * value size]``.  ``softcap > 0``: a score ``s = q . k * scale`` becomes ``softcap * tanh(s /
        softcap)``.  ``sink [heads]`` (float32): the softmax's denominator also holds ``exp(sink_h)``, a term with
        no key and no value that is neither scaled nor capped."""

    def qkv_norm_write(self, qkv, bias, step: StepTensors, kv: KvSlot | None, rotary: RotaryTable | None,
                       num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, norm_eps: float | None,
                       q_weight, k_weight, q_temp, q_out) -> None:
        """``qkv`` is the float32 projection ``[T, heads * head_dim + kv_heads * (head_dim + value_dim)]`` (or the
        slices of a split product; more columns behind these are not read) and ``bias`` its float32 bias or None.
        With ``norm_eps`` every head of q and k is divided by its root mean square over ``head_dim`` (eps inside
        the root) and, with ``q_weight`` / ``k_weight`` (float32 ``[head_dim]``), multiplied by it; THEN q and k are
        rotated (``rotary``); with ``q_temp = (coef, every)`` q at position p is multiplied by
        ``1 + coef * ln(floor((p + 1) / every) + 1)`` (``every`` a positive number).  k and v go to their pages (if ``kv``; values may have
        another size than keys) and q to ``q_out [T, heads * head_dim]`` in the set's dtype.  All float32."""
        raise NotImplementedError

    # -- norms around a sublayer, keys that are their own values, routed feed-forwards -----------------------------
    def norm_add_rmsnorm(self, delta, delta_weight, delta_eps: float, residual, weight, eps: float, out,
                         rows_index=None) -> None:
        """``d = sum of delta's terms`` (float32); ``residual += d * rsqrt(mean(d^2) + delta_eps) * delta_weight``
        (kept); ``out = cast(residual * rsqrt(mean(residual^2) + eps) * weight)``, everything in float32 up to the
        one cast.  ``delta``: None (nothing is added), a matrix, float32 slices or :class:`Terms`; with
        ``delta_weight`` None the sum is added as it is.  With ``rows_index`` only those rows are made and the
        residual stays as it is.  ``out`` None: only the residual is moved on."""
        raise NotImplementedError

    def qk_rope_norm_write(self, qk, bias, step: StepTensors, kv: KvSlot | None, rotary: RotaryTable | None,
                           num_heads: int, num_kv_heads: int, head_dim: int, norm_eps: float | None, q_out) -> None:
        """For layers whose values are their keys: ``qk`` is the projection ``[T, (heads + kv_heads) * head_dim]``
        (float32, or the float32 slices of a split product) and ``bias`` its float32 bias or None.  The key with
        its bias, before anything else is done to it, is stored as the value; q and k are rotated (``rotary``),
        then, with ``norm_eps`` not None, each head is divided by its root mean square over ``head_dim``; k goes to
        its page (if ``kv``) and q to ``q_out [T, heads * head_dim]`` in the set's dtype.  All arithmetic float32."""
        raise NotImplementedError

    def activation(self, x, kind: str = "silu", scale: float = 1.0, scaled_columns: int = 0):
        """A float32 matrix ``[T, n]`` out of ``x`` (float32, any row stride, or slices): ``act(x)`` with ``kind``
        ``"silu"`` or ``"none"``, the first ``scaled_columns`` columns also times ``scale``."""
        raise NotImplementedError

    def exp_gate_scan(self, log_in, log_forget, in_bias, forget_bias, cap: float, state, step: StepTensors):
        """Exponential gates with a running maximum, per head and request, float32:

        ``i = cap * tanh((log_in + in_bias) / cap)``; ``f = logsigmoid(cap * tanh((log_forget + forget_bias) / cap))``;
        ``m_t = max(f_t + m_(t-1), i_t)``; returns ``(keep, take, floor)``, each ``[T, heads]``:
        ``keep = exp(f + m_(t-1) - m_t)``, ``take = exp(i - m_t)``, ``floor = exp(-m_t)``.
        ``log_in, log_forget [T, heads]`` float32 (or slices); ``state [seats, heads]`` holds m (0 at a request's
        start) and is moved on by the step's tokens."""
        raise NotImplementedError

    def stabilized_readout(self, read, floor, heads: int, value_dim: int):
        """``read [T, heads * (value_dim + 1)]`` is the read-out of a recurrence whose last column per head is the
        normaliser ``n . q``: returns float32 ``[T, heads * value_dim]`` with head h of token t divided by
        ``max(|n . q|, floor[t, h]) + 1e-6``."""
        raise NotImplementedError

    def route_top(self, x, router, top: int, scoring: str = "sigmoid", groups: tuple[int, int] | None = None,
                  weight_scale: float = 1.0, extra_rows: int = 0, correction=None, normalise: bool = False):
        """The ``top`` experts of every token: logits ``x @ router.T`` (``router [experts, hidden]``) accumulated in
        float32 -> ``(ids [T, top] int32, weights [T, top] float32)``, ``weights`` the chosen experts' scores
        (``sigmoid(logit)``, not renormalised) times ``weight_scale``, the largest first, ties to the lower index.

        ``groups = (count, keep)``: the experts form ``count`` equal groups of neighbours; a group's score is the
        sum of its two largest scores (of its one score, for groups of one), and only experts of the ``keep`` groups
        with the largest scores (ties to the lower group) can be chosen.  With ``extra_rows`` the router matrix has
        that many more rows below the experts', which are no experts: their float32 logits ``[T, extra_rows]`` are
        returned as a third value (a gate that reads the same input, made in the same pass).

        ``scoring="softmax"``: the scores are a softmax over all experts' logits.  ``correction [experts]``
        (float32) is added to the scores for the choice only; the weights are the plain scores.  ``normalise``:
        the chosen scores are divided by their sum (+ 1e-20) before ``weight_scale``."""
        raise NotImplementedError

    def routed_swiglu(self, x, ids, weights, gate_up, down, scale_input: bool = True, limit: float | None = None,
                      identity: int = 0):
        """Every token through its chosen experts: ``gate_up [experts, 2 ff, hidden]`` (gate rows, then up rows),
        ``down [experts, hidden, ff]``; expert e of pair (t, j) computes ``down_e (silu(gate_e z) * (up_e z))`` with
        ``z = weights[t, j] * x[t]`` (``scale_input``) or on ``x[t]`` with the result times the weight.  With a
        ``limit`` the hidden activation is the capped form of :meth:`linear_glu`.  Returns
        float32 slices ``[top, T, hidden]`` whose sum over the first axis is the routed output.  With ``identity = n``
        ids ``experts .. experts + n - 1`` stand for experts that return their input: such a pair's slice row is
        ``weights[t, j] * x[t]`` (``scale_input`` False only)."""
        raise NotImplementedError

    def linear_glu(self, x, weight, limit: float | None = None, row_gate=None):
        """A gated hidden layer: ``weight = [Wg; Wu]`` stacked along the rows, ``g = x Wg^T``, ``u = x Wu^T``
        (float32 accumulators).  ``limit`` None: ``silu(g) * u``; a number: the capped form
        ``g' = min(g, limit)``, ``u' = clamp(u, -limit, limit)``, ``g' * sigmoid(1.702 g') * (u' + 1)``.
        ``row_gate`` (float32 ``[T]`` logits, any stride, or slices ``[S, T]``): row t also times
        ``sigmoid(row_gate[t])``.  Returns ``[T, rows / 2]`` in the set's dtype."""
        raise NotImplementedError

    def linear_act(self, x, weight, kind: str = "relu2"):
        """``act(x @ weight.T)`` in the set's dtype, the activation applied to the float32 accumulators:
        ``"relu2"`` is ``max(z, 0)^2``."""
        raise NotImplementedError

    # -- attention through a latent: one shared key/value row per token, queries folded into the latent's space ------
    def latent_kv_write(self, proj, step: StepTensors, kv: KvSlot | None, rotary: RotaryTable | None, q_rank: int,
                        q_norm, kv_rank: int, kv_norm, rot_dim: int, eps: float, q_latent_out) -> None:
        """``proj`` is the float32 projection ``[T, q_rank (+ kv_rank + rot_dim)]`` (or its slices).  Columns
        ``[0, q_rank)`` divided by their root mean square (``eps`` inside the root) times ``q_norm`` go to
        ``q_latent_out [T, q_rank]`` in the set's dtype.  With ``kv`` the next ``kv_rank`` columns, normed the same
        way with ``kv_norm``, and the last ``rot_dim`` columns, rotated by ``rotary`` at the token's position and not
        normed, are stored side by side as the token's one row ``[kv_rank + rot_dim]`` of ``kv.k``.  All float32
        up to the stores.  Without ``kv`` the projection has the query columns only."""
        raise NotImplementedError

    def latent_queries(self, q, up_keys, step: StepTensors, rotary: RotaryTable | None, num_heads: int, dim: int,
                       rot_dim: int):
        """``q`` is the float32 query projection ``[T, heads * (dim + rot_dim)]`` (or its slices), per head ``dim``
        plain columns and ``rot_dim`` columns to rotate; ``up_keys [heads, dim, kv_rank]`` maps a latent to a
        head's plain key.  Returns ``(folded [heads, T, kv_rank], rotated [T, heads, rot_dim])`` in the set's
        dtype: ``folded[h, t] = q_plain[t, h] @ up_keys[h]`` (so that ``folded . latent == q_plain . key``)."""
        raise NotImplementedError

    def latent_attention(self, folded, rotated, step: StepTensors, kv: KvSlot, num_heads: int, kv_rank: int,
                         rot_dim: int, scale: float, sink, out) -> None:
        """Causal softmax attention of every token over its request's rows ``[latent | rotated key part]`` of
        ``kv.k``, shared by all heads: score ``(folded[h, t] . latent_j + rotated[t, h] . part_j) * scale`` for every
        ``j <= position``; with ``sink [heads]`` (float32) the denominator also holds ``exp(sink_h)``;
        ``out[h, t] = sum_j weight_j latent_j`` (``[heads, T, kv_rank]``, the set's dtype).  Scores, softmax and the
        sum are float32."""
        raise NotImplementedError

    def latent_values(self, mixed, up_values, gate, num_heads: int, value_dim: int):
        """``mixed [heads, T, kv_rank]`` (what :meth:`latent_attention` left), ``up_values [heads, kv_rank,
        value_dim]`` -> ``[T, heads * value_dim]`` in the set's dtype: head h of token t is ``mixed[h, t] @
        up_values[h]`` times ``sigmoid(gate[t, h])`` (``gate`` float32 ``[T, heads]``, any stride, or slices; None:
        no gate)."""
        raise NotImplementedError

    # -- layer norm, gates, short convolutions and linear recurrences (layers with per-request state) --------
    # Where a float32 input is marked "or slices" it may also be ``[S, T, n]``, the slices of a split product
    # (:meth:`linear_split`) or a view of their columns: the op adds them up while it loads.
    def add_layernorm(self, delta, residual, weight, bias, eps: float, out, rows_index=None) -> None:
        """residual += delta (float32, kept); out = (residual - mean) / sqrt(var + eps) * weight + bias, with the
        variance the mean of the squared deviations.  ``delta``: None, ``[T, hidden]``, float32 slices
        ``[S, T, hidden]`` or :class:`Terms`.  With ``rows_index`` only those rows, residual kept."""
        raise NotImplementedError

    def kv_write(self, k, v, step: StepTensors, kv: KvSlot) -> None:
        """Store the new tokens' keys ``[T, kv_heads * head_dim]`` and values ``[T, kv_heads * value_dim]``
        (any float type, any row stride) in their pages: the write of layers that rotate nothing."""
        raise NotImplementedError

    def head_gate(self, x, logits, num_heads: int) -> None:
        """x ``[T, heads * d]`` in place: head h of token t times sigmoid(logits[t, h]) (float32 logits, or slices).
        With ``num_heads`` the number of columns (``d = 1``) the gate is element by element."""
        raise NotImplementedError

    def short_conv(self, x, weight, bias, state, step: StepTensors, activation: str = "silu", input_bias=None):
        """Causal convolution over time, per channel and per request: ``x [T, C]`` float32 (any row stride; or slices),
        ``weight [C, taps]`` whose last column multiplies the current token, ``state [seats, taps - 1, C]`` the
        request's last inputs (oldest first; zeros at a request's start), which the call moves on by the
        step's tokens.  Returns float32 ``[T, C]`` after the activation (``"silu"`` or ``"none"``).  ``input_bias [C]``
        (float32) is added to every input of the step before anything else (the state holds the sums; before a
        request's start the inputs are zeros, not the bias)."""
        raise NotImplementedError

    def linear_recurrence(self, rule: str, q, k, v, decay, write, state, step: StepTensors, heads: int, groups: int,
                          key_dim: int, value_dim: int, decay_rate=None, decay_bias=None, skip=None,
                          unit_column: bool = False):
        """A matrix state ``S [key_dim, value_dim]`` per head and request, moved on token by token in float32:

        ``S <- g S;  u = write-term;  S <- S + k u^T;  o = S^T q (+ skip * v)``

        Head h reads q and k of group ``h // (heads / groups)``.  ``q, k [T, groups * key_dim]``,
        ``v [T, heads * value_dim]``, ``decay, write [T, heads]`` (or slices), all float32 with any row stride.

        ``rule="delta"``: q and k are made unit vectors per head first (``x / sqrt(sum x^2 + 1e-6)``, q also
        times ``key_dim**-0.5``); ``g = exp(-exp(decay_rate) * softplus(decay + decay_bias))``;
        ``u = sigmoid(write) * (v - S^T k)`` with the decayed S.
        ``rule="ssd"``: ``dt = softplus(write + decay_bias)``; ``g = exp(-exp(decay_rate) * dt)``; ``u = dt * v``;
        ``skip [heads]`` adds ``skip_h * v`` to the read-out (``decay`` is not read).
        ``rule="gated"``: nothing is normalised; ``g = decay[t, h]`` as given, or with ``decay`` None the constant
        ``decay_rate[h]``; ``u = write[t, h] * v``, or ``v`` with ``write`` None.  With ``unit_column`` the state has
        one more column per head than ``v`` has elements (``value_dim`` counts it), whose value is 1 for every
        token: it carries ``n <- g n + write k`` and its read-out ``n . q`` is the last column of each head.

        ``state`` is ``[seats, heads, value_dim, key_dim]`` float32 (S transposed), read and written through
        each token's seat.  Returns float32 ``[T, heads * value_dim]``.  A set may overwrite ``q`` and ``k``
        (with their unit vectors): the caller hands over buffers it no longer needs."""
        raise NotImplementedError

    def gated_rmsnorm(self, x, gate, weight, eps: float, group: int, gate_first: bool, out,
                      activation: str = "silu") -> None:
        """Root-mean-square norm over groups of ``group`` neighbouring columns of ``x [T, n]`` (float32) with
        a gate (float32, or slices; written ``silu`` below, ``activation="sigmoid"`` makes it ``sigmoid(gate)``): ``gate_first``: ``norm(x * silu(gate)) * weight``; else ``norm(x) * weight * silu(gate)``.
        ``weight`` is float32 of ``n`` elements, or fewer, then repeated (``weight[column % len]``)."""
        raise NotImplementedError

    @abstractmethod
    def sample(self, logits, temperatures, uniforms, out_tokens) -> None:
        """Arg-max for rows with temperature <= 0, inverse-CDF draw at uniforms[row] otherwise."""

    def check_errors(self) -> None:
        """Raise if a kernel of an earlier launch reported a bad index (after a synchronise)."""
