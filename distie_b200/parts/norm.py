"""Norms: float32 statistics; each part also does the residual sum that precedes it, in the same kernel.

``rmsnorm``: formula of the reference (worker/src/inference/qwen2/model.py:85-90), the weight
applied after the cast back.  With an ``offset`` (a scale stored around zero: the norm multiplies by
``offset + weight``) the norm is float32 up to one cast at the end, and what it adds to the residual may
itself be a norm of a sublayer's output (:class:`~distie_b200.kernels.interface.Normed`): the sum, both
norms and the addition are one kernel.
``layernorm``: ``(x - mean) / sqrt(variance + eps) * weight + bias`` with the variance the mean of the
squared deviations, all in float32 up to the store.
"""

from __future__ import annotations

from ..config.model_spec import PartSpec
from ..kernels.interface import Normed, Terms
from .base import NORMS, BuildContext, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm:
    """params: ``eps``; optional ``name`` (what the tensor's name adds to the prefix, default ``"weight"``),
    ``offset`` (added to the stored scale; 0 when the checkpoint stores the scale itself) and ``exact`` (the norm
    is float32 up to the one cast of its output, scale included; an offset implies it).
    tensors: ``<prefix><name> [hidden]``."""

    def __init__(self, weight, eps: float, kernels, exact: bool = False) -> None:
        self.weight = weight
        self.eps = float(eps)
        self.kernels = kernels
        self.exact = exact  # float32 up to the one cast at the end (norm_add_rmsnorm) instead of the reference's order

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        role = "norm0" if float(spec.params.get("offset", 0.0)) else "norm"
        return [TensorSpec(spec.prefix + spec.params.get("name", "weight"), (hidden_size,), role)]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "RMSNorm":
        weight = ctx.weights.vector(spec.prefix + spec.params.get("name", "weight"))
        offset = float(spec.params.get("offset", 0.0))
        if offset:
            weight = weight + offset  # float32: exact for a scale stored in 16 bits, up to float32 rounding
        return cls(weight, spec.params["eps"], ctx.kernels, exact=bool(offset) or bool(spec.params.get("exact")))

    def pending(self, value) -> Normed:
        """``value`` (a sublayer's output) as something the next norm adds to the residual through this norm."""
        return Normed(value, self.weight, self.eps)

    def apply(self, delta, residual, out, rows=None) -> None:
        """``residual += delta`` (if any), ``out = norm(residual)``; with ``rows`` only those rows, residual kept."""
        if isinstance(delta, Normed):
            self.kernels.norm_add_rmsnorm(delta.value, delta.weight, delta.eps, residual, self.weight, self.eps, out, rows)
            return
        if self.exact:
            self.kernels.norm_add_rmsnorm(delta, None, 0.0, residual, self.weight, self.eps, out, rows)
            return
        if isinstance(delta, Terms):
            delta = delta.total()
        self.kernels.add_rmsnorm(delta, residual, self.weight, self.eps, out, rows)


@NORMS.register("layernorm")
class LayerNorm:
    """params: ``eps``; ``weight`` and ``bias``: what the tensors' names add to the prefix (defaults
    ``"weight"`` and ``"bias"``)."""

    def __init__(self, weight, bias, eps: float, kernels) -> None:
        self.weight = weight
        self.bias = bias
        self.eps = float(eps)
        self.kernels = kernels

    @staticmethod
    def _names(spec: PartSpec) -> tuple[str, str]:
        return spec.prefix + spec.params.get("weight", "weight"), spec.prefix + spec.params.get("bias", "bias")

    @classmethod
    def tensor_specs(cls, spec: PartSpec, hidden_size: int) -> list[TensorSpec]:
        weight, bias = cls._names(spec)
        return [TensorSpec(weight, (hidden_size,), "norm"), TensorSpec(bias, (hidden_size,), "bias")]

    @classmethod
    def build(cls, spec: PartSpec, ctx: BuildContext) -> "LayerNorm":
        weight, bias = cls._names(spec)
        return cls(ctx.weights.vector(weight), ctx.weights.vector(bias), spec.params["eps"], ctx.kernels)

    def apply(self, delta, residual, out, rows=None) -> None:
        """``residual += delta`` (if any; a :class:`Terms` is summed in the kernel), ``out = norm(residual)``."""
        self.kernels.add_layernorm(delta, residual, self.weight, self.bias, self.eps, out, rows)
