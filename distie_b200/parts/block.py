"""Arrangements of parts in a block.

``pre_norm``: the reference's decoder layer (worker/src/inference/qwen2/model.py:
247-249): ``h += mixer(norm_in(h))``; ``h += ff(norm_post(h))``.  The sums are
float32 and are done by the norm kernel that follows them, so a block leaves its
feed-forward output pending on the stream.

``sandwich``: a norm before and after each sublayer: ``h += norm_b(mixer(norm_a(h)))``;
``h += norm_d(ff(norm_c(h)))``.  The norm of a sublayer's output, the addition to the float32 residual and
the norm before the next sublayer are one kernel: a sublayer's output stays pending as a
:class:`~distie_b200.kernels.interface.Normed`.  A feed-forward of kind ``none`` (with its two norms) is left out.

``parallel``: one norm, and mixer and feed-forward both read its output:
``h += mixer(norm(h)) + ff(norm(h))``.  Both outputs stay pending as one weighted sum, which the
next block's norm kernel adds to the float32 residual.
"""

from __future__ import annotations

import torch

from ..config.model_spec import LayerSpec
from ..kernels.interface import Terms
from .base import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Branches, BuildContext, LayerRun, ResidualStream, TensorSpec, build_part


@BLOCKS.register("pre_norm")
class PreNormBlock:
    """norms: ``input`` (before the mixer) and ``post_mixer`` (before the feed-forward).  A layer whose feed-forward
    is of kind ``none`` may leave ``post_mixer`` out: the mixer's output then stays pending for the next norm."""

    def __init__(self, norm_in, mixer, norm_post, feed_forward, dtype) -> None:
        self.norm_in = norm_in
        self.mixer = mixer
        self.norm_post = norm_post
        self.feed_forward = feed_forward
        self.dtype = dtype

    @property
    def graph_safe(self) -> bool:
        """False when a part reads host-side batch data, which a captured step cannot replay."""
        return all(getattr(part, "graph_safe", True) for part in (self.mixer, self.feed_forward))

    @classmethod
    def tensor_specs(cls, layer: LayerSpec, hidden_size: int) -> list[TensorSpec]:
        return (
            NORMS.get(layer.norms["input"].kind).tensor_specs(layer.norms["input"], hidden_size)
            + MIXERS.get(layer.mixer.kind).tensor_specs(layer.mixer, hidden_size)
            + (NORMS.get(layer.norms["post_mixer"].kind).tensor_specs(layer.norms["post_mixer"], hidden_size)
               if "post_mixer" in layer.norms else [])
            + FEED_FORWARDS.get(layer.feed_forward.kind).tensor_specs(layer.feed_forward, hidden_size)
        )

    @classmethod
    def build(cls, layer: LayerSpec, ctx: BuildContext) -> "PreNormBlock":
        if "post_mixer" not in layer.norms and layer.feed_forward.kind != "none":
            raise ValueError("a pre_norm layer with a feed-forward needs the norm 'post_mixer'")
        return cls(
            build_part(NORMS, layer.norms["input"], ctx),
            build_part(MIXERS, layer.mixer, ctx),
            build_part(NORMS, layer.norms["post_mixer"], ctx) if "post_mixer" in layer.norms else None,
            build_part(FEED_FORWARDS, layer.feed_forward, ctx),
            ctx.dtype,
        )

    def forward(self, stream: ResidualStream, run: LayerRun) -> None:
        residual = stream.residual
        x = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        self.norm_in.apply(stream.pending, residual, x)
        mixed = self.mixer.forward(x, run)
        if self.norm_post is None:  # no feed-forward: the next norm adds the mixer's output to the residual
            stream.pending = mixed
            return
        self.norm_post.apply(mixed, residual, x)
        stream.pending = self.feed_forward.forward(x, run)


@BLOCKS.register("parallel")
class ParallelBlock:
    """norms: ``input`` only.  A feed-forward of kind ``none`` adds nothing."""

    def __init__(self, norm_in, mixer, feed_forward, dtype, kernels=None) -> None:
        self.norm_in = norm_in
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.dtype = dtype
        self.kernels = kernels

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", True) for part in (self.mixer, self.feed_forward))

    @classmethod
    def tensor_specs(cls, layer: LayerSpec, hidden_size: int) -> list[TensorSpec]:
        return (
            NORMS.get(layer.norms["input"].kind).tensor_specs(layer.norms["input"], hidden_size)
            + MIXERS.get(layer.mixer.kind).tensor_specs(layer.mixer, hidden_size)
            + FEED_FORWARDS.get(layer.feed_forward.kind).tensor_specs(layer.feed_forward, hidden_size)
        )

    @classmethod
    def build(cls, layer: LayerSpec, ctx: BuildContext) -> "ParallelBlock":
        return cls(
            build_part(NORMS, layer.norms["input"], ctx),
            build_part(MIXERS, layer.mixer, ctx),
            build_part(FEED_FORWARDS, layer.feed_forward, ctx),
            ctx.dtype,
            ctx.kernels,
        )

    def forward(self, stream: ResidualStream, run: LayerRun) -> None:
        residual = stream.residual
        x = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        self.norm_in.apply(stream.pending, residual, x)
        # What the sublayers share of the step (where each request's tokens lie) is made before they part.
        prepare = getattr(self.kernels, "prepare_step", None)
        if prepare is not None:
            prepare(run.step)
        # The mixer's branches (one, or the two of a pair side by side) and the feed-forward read x and nothing of
        # one another: in a step of few tokens they run side by side.
        jobs = list(self.mixer.branches(x, run)) if hasattr(self.mixer, "branches") else [lambda: self.mixer.forward(x, run)]
        if not isinstance(self.feed_forward, FEED_FORWARDS.get("none")):
            jobs.append(lambda: self.feed_forward.forward(x, run))
        outputs = Branches.run(jobs, x.shape[0], x.device)
        pending = Terms.of(outputs[0])
        for more in outputs[1:]:
            pending = pending + Terms.of(more)
        stream.pending = pending


@BLOCKS.register("sandwich")
class SandwichBlock:
    """norms: ``input`` and ``mixer_out`` around the mixer, ``post_mixer`` and ``ff_out`` around the feed-forward
    (the latter two only when the layer has a feed-forward).  The norms are of kind ``rmsnorm``."""

    def __init__(self, norm_in, mixer, norm_mixer_out, norm_post, feed_forward, norm_ff_out, dtype) -> None:
        self.norm_in, self.mixer, self.norm_mixer_out = norm_in, mixer, norm_mixer_out
        self.norm_post, self.feed_forward, self.norm_ff_out = norm_post, feed_forward, norm_ff_out
        self.dtype = dtype

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", True) for part in (self.mixer, self.feed_forward) if part is not None)

    @staticmethod
    def _has_ff(layer: LayerSpec) -> bool:
        return layer.feed_forward.kind != "none"

    @classmethod
    def _norm_names(cls, layer: LayerSpec) -> list[str]:
        return ["input", "mixer_out"] + (["post_mixer", "ff_out"] if cls._has_ff(layer) else [])

    @classmethod
    def tensor_specs(cls, layer: LayerSpec, hidden_size: int) -> list[TensorSpec]:
        specs = []
        for name in cls._norm_names(layer):
            specs += NORMS.get(layer.norms[name].kind).tensor_specs(layer.norms[name], hidden_size)
        specs += MIXERS.get(layer.mixer.kind).tensor_specs(layer.mixer, hidden_size)
        if cls._has_ff(layer):
            specs += FEED_FORWARDS.get(layer.feed_forward.kind).tensor_specs(layer.feed_forward, hidden_size)
        return specs

    @classmethod
    def build(cls, layer: LayerSpec, ctx: BuildContext) -> "SandwichBlock":
        norms = {name: build_part(NORMS, layer.norms[name], ctx) for name in cls._norm_names(layer)}
        for name, norm in norms.items():
            if not hasattr(norm, "pending") and name in ("mixer_out", "ff_out"):
                raise ValueError(f"the '{name}' norm of a sandwich block must be able to stay pending (kind rmsnorm)")
        feed_forward = build_part(FEED_FORWARDS, layer.feed_forward, ctx) if cls._has_ff(layer) else None
        return cls(norms["input"], build_part(MIXERS, layer.mixer, ctx), norms["mixer_out"], norms.get("post_mixer"),
                   feed_forward, norms.get("ff_out"), ctx.dtype)

    def forward(self, stream: ResidualStream, run: LayerRun) -> None:
        residual = stream.residual
        x = torch.empty(residual.shape, dtype=self.dtype, device=residual.device)
        self.norm_in.apply(stream.pending, residual, x)
        mixed = self.norm_mixer_out.pending(self.mixer.forward(x, run))
        if self.feed_forward is None:
            stream.pending = mixed
            return
        self.norm_post.apply(mixed, residual, x)
        stream.pending = self.norm_ff_out.pending(self.feed_forward.forward(x, run))
