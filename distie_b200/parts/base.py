"""Interfaces and registries of the parts a block is put together from.

A part is built from a :class:`~distie_b200.config.model_spec.PartSpec` (its
constants and the prefix of its tensors) and a :class:`BuildContext` (the kernel
set, the hidden width, the loaded weights).  No part knows which model it is in.

============== ==============================================================
kind of part   what it must offer
============== ==============================================================
norm           ``tensor_specs``, ``build``, ``apply(delta, residual, out, rows=None)``
position       ``build``; ``rotary_table()`` for the fused kernel, or ``None``
               and an ``apply(qkv, step, ...)`` of its own
mixer          ``tensor_specs``, ``build``, ``cache_need``, ``state_need``,
               ``forward(x, run) -> delta``
feed-forward   ``tensor_specs``, ``build``, ``forward(x, run) -> delta``
block          ``tensor_specs``, ``build``, ``forward(stream, run)``
============== ==============================================================

``forward`` of a mixer or feed-forward takes the normalised activations ``[T,
hidden]`` of the step's tokens and returns what is to be added to the residual
stream: ``[T, hidden]``, float32 slices ``[S, T, hidden]`` whose sum it is (what
``KernelSet.linear_split`` returns; the norm that follows adds them up), or
:class:`~distie_b200.kernels.interface.Terms`, a weighted sum of such tensors.  The :class:`LayerRun` tells a mixer everything about the step: the
tokens' positions and requests, its cache slot and its per-request state.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Sequence

import torch

from ..config.model_spec import PartSpec
from ..kernels.interface import KernelSet, KvSlot, Normed, StepTensors, Terms


# -- what parts declare --------------------------------------------------------
@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part reads from the checkpoint.  ``role`` decides conversion and random init:

    ``matrix``  2-D weight of a product (engine dtype; a float32-stored one stays float32)
    ``table``   embedding table (like ``matrix``)
    ``bias``    vector added to a product (kept in float32 on the device)
    ``norm``    scale of a norm (float32 on the device; random mode writes ones)
    ``norm0``   scale of a norm that is stored around zero (the norm multiplies by 1 + it; random mode writes zeros)
    """

    name: str
    shape: tuple[int, ...]
    role: str = "matrix"


@dataclass(frozen=True)
class CacheNeed:
    """Keys and values in pages.  Layers with equal needs share a group (pool, tables)."""

    num_kv_heads: int
    head_dim: int
    window: int | None = None  # None: every key is kept; n: only the last n positions are read
    chunk: int | None = None   # n: a token reads only keys of its own chunk of n positions (counted from 0)
    value_dim: int | None = None  # size of a value when it differs from head_dim
    keep_first: int = 0        # beside a window: the request's first n positions stay readable for good
    values_in_keys: bool = False  # a value is the first value_dim columns of its key's row: nothing is stored twice

    @property
    def v_dim(self) -> int:
        return int(self.value_dim or self.head_dim)

    @property
    def row_elements(self) -> int:
        """Elements one token holds per kv head in a slot of this group."""
        return self.head_dim if self.values_in_keys else self.head_dim + self.v_dim


@dataclass(frozen=True)
class StateNeed:
    """State of fixed size per request (one slot per seat), zeroed when a request starts.

    A mixer's ``state_need`` returns one of these, or a dict of them by name when it keeps several
    tensors (a matrix state and the last inputs of a short convolution, say); ``LayerRun.state`` is then
    a dict of tensors under the same names."""

    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


# -- what parts are given ------------------------------------------------------
@dataclass
class BuildContext:
    kernels: KernelSet
    hidden_size: int
    weights: Any  # distie_b200.weights.loader.WeightStore

    @property
    def dtype(self) -> torch.dtype:
        return self.kernels.dtype

    @property
    def device(self) -> torch.device:
        return self.kernels.device


@dataclass(frozen=True)
class SeqSlice:
    """One request's share of a step, on the host: tokens [start, start + q_len) of the batch."""

    seat: int
    start: int
    q_len: int
    past_len: int


@dataclass
class LayerRun:
    """Everything one call of the run order may look at."""

    step: StepTensors
    seqs: Sequence[SeqSlice]
    kv: KvSlot | None = None
    state: Any = None  # [seats, *StateNeed.shape] of this call's slot, or a dict of such tensors by name
    writes_cache: bool = True
    extras: dict = field(default_factory=dict)


class ResidualStream:
    """The float32 residual ``[T, hidden]`` and a delta that is still to be added.

    Keeping the delta pending lets the next norm do the sum and the normalisation
    in one kernel; ``settle`` performs the sum for a consumer that wants the plain
    residual.
    """

    def __init__(self, residual: torch.Tensor, pending: torch.Tensor | None = None) -> None:
        self.residual = residual
        self.pending = pending

    def settle(self) -> torch.Tensor:
        if isinstance(self.pending, Normed):  # a sublayer's output that joins the residual through a norm
            value = ResidualStream(torch.zeros_like(self.residual), self.pending.value).settle()
            unit = value * torch.rsqrt((value * value).mean(-1, keepdim=True) + self.pending.eps)
            self.residual.add_(unit * self.pending.weight)
            self.pending = None
        if self.pending is not None:
            if isinstance(self.pending, Terms):
                delta = self.pending.total()
            else:
                delta = self.pending.sum(0) if self.pending.dim() == 3 else self.pending  # slices of a split product
            self.residual.add_(delta.to(torch.float32))
            self.pending = None
        return self.residual


class Branches:
    """Sublayers of a block that read the same input and do not read one another: run side by side.

    On a CUDA device a step of few tokens is a chain of short kernels, each waiting for the one before; the
    branches of a parallel block (two mixers and a feed-forward) are independent chains, so each gets a stream
    of its own between a fork after the block's norm and a join before the next kernel of the main stream.
    A captured decode step records the fork and the join as edges of its graph.  Every tensor a branch makes
    and hands back is read only after the join and before the next fork, and what it frees returns to its own
    stream's pool, so no block of memory is reused while another stream may still read it.  Steps of many tokens
    fill the machine with every kernel and stay on one stream.
    """

    SMALL_STEP = 64
    _side: dict = {}

    @classmethod
    def run(cls, jobs, tokens: int, device: torch.device) -> list:
        if len(jobs) < 2 or device.type != "cuda" or tokens > cls.SMALL_STEP:
            return [job() for job in jobs]
        streams = cls._side.setdefault(str(device), [])
        while len(streams) < len(jobs) - 1:
            streams.append(torch.cuda.Stream(device=device))
        main = torch.cuda.current_stream(device)
        results = [None] * len(jobs)
        for index, job in enumerate(jobs[1:], start=1):
            side = streams[index - 1]
            side.wait_stream(main)
            with torch.cuda.stream(side):
                results[index] = job()
        results[0] = jobs[0]()
        for side in streams[: len(jobs) - 1]:
            main.wait_stream(side)
        return results


# -- registries ---------------------------------------------------------------
class Registry:
    def __init__(self, what: str) -> None:
        self.what = what
        self._kinds: dict[str, Any] = {}

    def register(self, kind: str, cls: Any = None) -> Callable | Any:
        if cls is None:
            def wrap(inner):
                self._kinds[kind] = inner
                return inner
            return wrap
        self._kinds[kind] = cls
        return cls

    def unregister(self, kind: str) -> None:
        self._kinds.pop(kind, None)

    def get(self, kind: str) -> Any:
        try:
            return self._kinds[kind]
        except KeyError:
            raise KeyError(f"unknown {self.what} {kind!r}; registered: {', '.join(sorted(self._kinds))}") from None

    def kinds(self) -> tuple[str, ...]:
        return tuple(sorted(self._kinds))


MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
NORMS = Registry("norm")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block arrangement")


def build_part(registry: Registry, spec: PartSpec, ctx: BuildContext):
    return registry.get(spec.kind).build(spec, ctx)
