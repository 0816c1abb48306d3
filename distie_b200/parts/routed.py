"""Routed feed-forward: every token goes through a few of many small gated experts, and through a shared one.

``routed_swiglu``: router scores ``s = sigmoid(W_router h)`` from float32 logits; the ``top`` experts with the
largest scores are chosen (ties to the lower index) and weighted by their scores as they are (times
``weight_scale``); with ``weight_on="input"`` the weight multiplies what the expert reads, ``sum_e expert_e(s_e h)``,
with ``"output"`` what it returns.  With ``groups = (count, keep)`` the experts form ``count`` equal groups of
neighbours, a group's score is the sum of its two largest scores, and only experts of the ``keep`` best groups can
be chosen.  An expert is ``down(silu(gate h) * (up h))`` or, with a ``limit``, the capped form
``g = min(gate h, limit)``, ``u = clamp(up h, -limit, limit)``, ``down(g * sigmoid(1.702 g) * (u + 1))``.
A shared expert of the same form (with a limit of its own) runs for every token and is added; with
``shared_gate`` it is first multiplied by ``sigmoid(w_sg . h)``, one number per token, whose logit is made
in the router's pass (``w_sg`` is one more row below the router's).  ``scoring="softmax"`` takes the scores as a
softmax over all router outputs; ``correction`` names a vector (``[router outputs]``) that is added to the scores for
the choice only; ``normalise`` divides the chosen scores by their sum (+ 1e-20); with ``identity = n`` the router has
``n`` more outputs than there are experts, which stand for experts without tensors that return their input.  The output stays a sum still to be done
(the routed slices and the shared expert's), which the norm kernel that follows adds up.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from ..kernels.interface import Terms
from .base import FEED_FORWARDS, Branches, BuildContext, LayerRun, TensorSpec
from .linear import fuse_rows


@FEED_FORWARDS.register("routed_swiglu")
class RoutedSwiGlu:
    """params: ``experts``, ``top``, ``intermediate_size``, ``shared_size`` (None: no shared expert), optional
    ``weight_on`` (``"input"``, default, or ``"output"``), ``weight_scale`` (default 1), ``groups`` (``(count,
    keep)`` or None), ``limit`` and ``shared_limit`` (None: SwiGLU), ``shared_gate`` (None, or what the name of
    the shared expert's gate vector adds to ``shared.``), ``scoring`` (``"sigmoid"``, default, or ``"softmax"``),
    ``correction`` (None, or the name of the vector added to the scores for the choice), ``normalise`` (bool) and
    ``identity`` (0: how many router outputs behind the experts' return their input).
    tensors (prefix +): ``router [experts + identity, hidden]``; ``<correction> [experts + identity]``; ``e<j>.gate, e<j>.up [ff, hidden]``, ``e<j>.down [hidden, ff]``;
    ``shared.gate, shared.up, shared.down``; ``shared.<shared_gate> [1, hidden]``."""

    graph_safe = True

    def __init__(self, router, gate_up, down, shared_gate_up, shared_down, prm: dict, kernels) -> None:
        self.router, self.gate_up, self.down = router, gate_up, down
        self.shared_gate_up, self.shared_down = shared_gate_up, shared_down
        self.experts, self.top = int(prm["experts"]), int(prm["top"])
        self.scale_input = prm.get("weight_on", "input") == "input"
        self.weight_scale = float(prm.get("weight_scale", 1.0))
        self.groups = tuple(int(v) for v in prm["groups"]) if prm.get("groups") else None
        self.limit = float(prm["limit"]) if prm.get("limit") is not None else None
        self.shared_limit = float(prm["shared_limit"]) if prm.get("shared_limit") is not None else None
        self.gated_shared = bool(prm.get("shared_gate")) and shared_gate_up is not None  # the gate's row lies below the router's
        self.scoring = prm.get("scoring", "sigmoid")
        self.normalise = bool(prm.get("normalise"))
        self.identity = int(prm.get("identity") or 0)
        self.correction = None  # set by build
        self.kernels = kernels

    @staticmethod
    def _check(prm) -> None:
        experts, top = int(prm["experts"]), int(prm["top"])
        identity = int(prm.get("identity") or 0)
        if experts < 1 or top < 1 or identity < 0 or top > experts + identity or top > 32:
            raise ValueError(f"experts {experts} (+ {identity} that return their input), top {top}: 1 <= top <= min(outputs, 32)")
        if prm.get("scoring", "sigmoid") not in ("sigmoid", "softmax"):
            raise ValueError(f"scoring {prm['scoring']!r}: 'sigmoid' or 'softmax'")
        if (identity or prm.get("correction")) and (prm.get("groups") or prm.get("shared_gate")):
            raise ValueError("identity experts and a correction do not go with groups or a gated shared expert")
        if identity and prm.get("weight_on", "input") != "output":
            raise ValueError("identity experts go with weight_on='output'")
        if prm.get("weight_on", "input") not in ("input", "output"):
            raise ValueError(f"weight_on {prm['weight_on']!r}: 'input' or 'output'")
        if prm.get("groups"):
            count, keep = (int(v) for v in prm["groups"])
            if count < 1 or experts % count or not 1 <= keep <= count or top > keep * (experts // count):
                raise ValueError(f"groups {prm['groups']!r}: count divides experts ({experts}), 1 <= keep <= count, "
                                 f"top ({top}) <= the experts of the kept groups")
        for key in ("limit", "shared_limit"):
            if prm.get(key) is not None and float(prm[key]) <= 0:
                raise ValueError(f"{key} must be positive, got {prm[key]}")
        if prm.get("shared_gate") and prm.get("shared_size") is None:
            raise ValueError("shared_gate without a shared expert")

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        cls._check(spec.params)
        p, prm = spec.prefix, spec.params
        ff = int(prm["intermediate_size"])
        specs = []
        for e in range(int(prm["experts"])):
            specs += [TensorSpec(f"{p}e{e}.gate", (ff, hidden_size)), TensorSpec(f"{p}e{e}.up", (ff, hidden_size)),
                      TensorSpec(f"{p}e{e}.down", (hidden_size, ff))]
        outputs = int(prm["experts"]) + int(prm.get("identity") or 0)
        specs.append(TensorSpec(p + "router", (outputs, hidden_size)))
        if prm.get("correction"):
            specs.append(TensorSpec(p + prm["correction"], (outputs,), "bias"))
        if prm.get("shared_size") is not None:
            shared = int(prm["shared_size"])
            specs += [TensorSpec(p + "shared.gate", (shared, hidden_size)), TensorSpec(p + "shared.up", (shared, hidden_size)),
                      TensorSpec(p + "shared.down", (hidden_size, shared))]
            if prm.get("shared_gate"):
                specs.append(TensorSpec(f"{p}shared.{prm['shared_gate']}", (1, hidden_size)))
        return specs

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "RoutedSwiGlu":
        cls._check(spec.params)
        p, prm, w = spec.prefix, spec.params, ctx.weights
        experts = range(int(prm["experts"]))
        gate_up = torch.stack([fuse_rows([w.matrix(f"{p}e{e}.gate"), w.matrix(f"{p}e{e}.up")]) for e in experts]).contiguous()
        down = torch.stack([w.matrix(f"{p}e{e}.down") for e in experts]).contiguous()
        shared_gate_up = shared_down = None
        if prm.get("shared_size") is not None:
            shared_gate_up = fuse_rows([w.matrix(p + "shared.gate"), w.matrix(p + "shared.up")])
            shared_down = w.matrix(p + "shared.down")
        router = w.matrix(p + "router")
        if prm.get("shared_gate") and shared_gate_up is not None:
            router = fuse_rows([router, w.matrix(f"{p}shared.{prm['shared_gate']}")])
        part = cls(router, gate_up, down, shared_gate_up, shared_down, dict(prm), ctx.kernels)
        if prm.get("correction"):
            part.correction = w.vector(p + prm["correction"])
        return part

    def forward(self, x: torch.Tensor, run: LayerRun):
        k = self.kernels
        plain = self.groups is None and self.weight_scale == 1.0 and self.limit is None and not self.gated_shared

        def routed():
            if self.scoring != "sigmoid" or self.correction is not None or self.normalise or self.identity:
                ids, weights = k.route_top(x, self.router, self.top, self.scoring, None, self.weight_scale, 0,
                                           self.correction, self.normalise)
                return k.routed_swiglu(x, ids, weights, self.gate_up, self.down, self.scale_input, self.limit, self.identity)
            if plain:
                ids, weights = k.route_top(x, self.router, self.top, "sigmoid")
                return k.routed_swiglu(x, ids, weights, self.gate_up, self.down, self.scale_input)
            ids, weights = k.route_top(x, self.router, self.top, "sigmoid", self.groups, self.weight_scale)
            return k.routed_swiglu(x, ids, weights, self.gate_up, self.down, self.scale_input, self.limit)

        def shared(row_gate=None):
            if self.shared_limit is None and row_gate is None:
                return k.linear_split(k.linear_swiglu(x, self.shared_gate_up), self.shared_down)
            return k.linear_split(k.linear_glu(x, self.shared_gate_up, self.shared_limit, row_gate), self.shared_down)

        if self.shared_gate_up is None:
            return Terms.of(routed())
        if self.gated_shared:
            # The shared expert waits for its gate, which the router's pass makes: the two run after one another.
            ids, weights, gate = k.route_top(x, self.router, self.top, "sigmoid", self.groups, self.weight_scale, 1)
            experts = k.routed_swiglu(x, ids, weights, self.gate_up, self.down, self.scale_input, self.limit)
            return Terms.of(experts) + Terms.of(shared(gate))
        # The routed experts and the shared one read the same input and nothing of one another: in a step of few
        # tokens, where each is a chain of short kernels, they run side by side.
        both = Branches.run([routed, shared], x.shape[0], x.device)
        return Terms.of(both[0]) + Terms.of(both[1])
