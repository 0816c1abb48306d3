"""Dense feed-forwards, no biases: SwiGLU ``down(silu(gate(x)) * up(x))`` and ``activated`` ``down(act(up(x)))``.

Formula of the reference (worker/src/inference/qwen2/model.py:228-236).  Gate and
up are one product against the row-stacked weight ``[2 * inter, hidden]``.
``none`` is the feed-forward of a layer that has none: it declares nothing and adds nothing.
"""

from __future__ import annotations

import torch

from ..config.model_spec import PartSpec
from .base import FEED_FORWARDS, BuildContext, LayerRun, TensorSpec
from .linear import Linear, fuse_rows


@FEED_FORWARDS.register("swiglu")
class SwiGluFeedForward:
    """params: ``intermediate_size``; optional ``names``: what the names of the gate, up and down matrices add to
    the prefix (default ``gate_proj.weight``, ``up_proj.weight``, ``down_proj.weight``)."""

    _NAMES = ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    def __init__(self, gate_up: Linear, down: Linear, inter: int, kernels) -> None:
        self.gate_up = gate_up
        self.down = down
        self.inter = inter
        self.kernels = kernels

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        p, inter = spec.prefix, int(spec.params["intermediate_size"])
        gate, up, down = spec.params.get("names", cls._NAMES)
        return [
            TensorSpec(p + gate, (inter, hidden_size)),
            TensorSpec(p + up, (inter, hidden_size)),
            TensorSpec(p + down, (hidden_size, inter)),
        ]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "SwiGluFeedForward":
        p, w = spec.prefix, ctx.weights
        gate, up, down = spec.params.get("names", cls._NAMES)
        gate_up = fuse_rows([w.matrix(p + gate), w.matrix(p + up)])
        return cls(
            Linear(gate_up, None, ctx.kernels),
            Linear(w.matrix(p + down), None, ctx.kernels),
            int(spec.params["intermediate_size"]),
            ctx.kernels,
        )

    def forward(self, x: torch.Tensor, run: LayerRun) -> torch.Tensor:
        # The down product's float32 slices are summed by the norm that follows (or by the stream).
        return self.kernels.linear_split(self.kernels.linear_swiglu(x, self.gate_up.weight), self.down.weight)


@FEED_FORWARDS.register("activated")
class ActivatedFeedForward:
    """``down(act(up(x)))`` with the activation on the product's float32 accumulators.  params:
    ``intermediate_size``, ``activation`` (``"relu2"``: the square of ReLU); optional ``names``: what the names of
    the up and down matrices add to the prefix (default ``up_proj.weight``, ``down_proj.weight``)."""

    _NAMES = ("up_proj.weight", "down_proj.weight")
    _ACTIVATIONS = ("relu2",)

    def __init__(self, up: torch.Tensor, down: torch.Tensor, activation: str, kernels) -> None:
        self.up, self.down, self.activation, self.kernels = up, down, activation, kernels

    @classmethod
    def _check(cls, spec: PartSpec) -> None:
        if spec.params.get("activation") not in cls._ACTIVATIONS:
            raise ValueError(f"activation {spec.params.get('activation')!r}: one of {cls._ACTIVATIONS}")

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        cls._check(spec)
        p, inter = spec.prefix, int(spec.params["intermediate_size"])
        up, down = spec.params.get("names", cls._NAMES)
        return [TensorSpec(p + up, (inter, hidden_size)), TensorSpec(p + down, (hidden_size, inter))]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "ActivatedFeedForward":
        cls._check(spec)
        p, w = spec.prefix, ctx.weights
        up, down = spec.params.get("names", cls._NAMES)
        return cls(w.matrix(p + up), w.matrix(p + down), spec.params["activation"], ctx.kernels)

    def forward(self, x: torch.Tensor, run: LayerRun) -> torch.Tensor:
        return self.kernels.linear_split(self.kernels.linear_act(x, self.up, self.activation), self.down)


@FEED_FORWARDS.register("none")
class NoFeedForward:
    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        return []

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "NoFeedForward":
        return cls()

    def forward(self, x: torch.Tensor, run: LayerRun):
        return None
