"""Interfaces of the parts a layer is put together from.

A part is built from a :class:`~lightllm_b200.config.PartSpec` as ``cls(prefix, **params)``:
every size and constant is a parameter, and no part knows which model it is in.  It lists the
checkpoint tensors it reads (:meth:`Part.weight_specs`), receives them already on the device in
:meth:`Part.bind`, and then runs on the GPU.

Roles and what each must provide:

``norm``       ``forward(residual[T, D] float32, ctx) -> x[T, D]`` in the compute dtype, and
               ``forward_rows(residual, rows[R] int32, ctx) -> x[R, D]``.
``mixer``      ``cache_spec() -> CacheSpec | None`` and
               ``forward(x[T, D], residual[T, D] float32, ctx, cache)``, which **adds** its output
               into ``residual`` in place.  ``cache`` is a :class:`CacheView` of the planes the
               layout gave this run of the layer, or ``None`` if it asked for nothing.
``ffn``        ``forward(x[T, D], residual[T, D] float32, ctx)``, adding into ``residual``.
``position``   ``rotary_table() -> (inv_freq, rotary_dim, interleaved) | None`` for encodings the
               fused rotation kernel can apply, else ``apply(q, k, positions) -> (q, k)``.
``embedding``  ``forward(token_ids[T] int32, ctx) -> residual[T, D] float32``.
``head``       ``forward(x[R, D], ctx) -> logits[R, V] float32``.

The residual stream is float32 in both precisions, so the residual sum is exact to float.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..cache import CacheSpec
from ..weights import WeightSpec


class Part:
    role = "part"
    # True when forward() only launches kernels whose arguments are fixed by the step's counts; a model of
    # such parts has its decode steps captured in CUDA graphs.  Parts that branch on the host say False.
    graph_safe = False
    # True when forward() takes a LazyNorm in place of the normalised tensor.
    accepts_lazy_norm = False

    def weight_specs(self) -> List[WeightSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype, device: torch.device) -> None:
        """Take this part's tensors out of ``tensors`` (by the names it declared)."""

    def children(self) -> List["Part"]:
        return []

    def prepare(self, ctx, cache=None) -> None:
        """Called for every run entry before the step's metadata is copied to the device: the place to make
        index arrays with ``ctx.stage`` / ``ctx.tiles`` so that they share that copy (and, for CUDA graphs,
        to append to ``ctx.shape_key`` whatever else the launches will depend on).

        A part whose preparation only depends on its own constants (not on its cache planes) may set
        ``prepare_key`` to a hashable value of them: of the parts of a model with equal keys only the first is
        called in a step."""

    prepare_key = None


class LazyNorm:
    """The normalised input of a mixer, feed-forward or head, not yet computed.

    A block hands this to parts that set ``accepts_lazy_norm``: they may fold the norm into their
    first kernel (``fusable()`` gives the weight and eps of an RMSNorm) or ask for the tensor
    (``materialize()``).  ``rows`` selects rows of the residual stream (the head's wanted rows)."""

    def __init__(self, residual: torch.Tensor, norm: "Norm", ctx=None, rows: Optional[torch.Tensor] = None):
        self.residual, self.norm, self.ctx, self.rows = residual, norm, ctx, rows
        self._value = None

    @property
    def num_rows(self) -> int:
        return self.rows.numel() if self.rows is not None else self.residual.shape[0]

    def fusable(self):
        f = getattr(self.norm, "rms_parameters", None)
        return f() if f is not None else None

    def materialize(self) -> torch.Tensor:
        if self._value is None:
            if self.rows is not None:
                self._value = self.norm.forward_rows(self.residual, self.rows, self.ctx)
            else:
                self._value = self.norm.forward(self.residual, self.ctx)
        return self._value


@dataclass
class CacheView:
    """The cache planes of one run of a layer.

    ``k``, ``v``: ``[pages * page_size, kv_heads, head_dim]`` or ``None``; ``group`` indexes
    ``ctx.slot_mapping`` and ``ctx.block_tables``; ``state``: ``[max_seqs, *shape]`` or ``None``,
    indexed by ``Span.slot``; ``writes`` is False when the planes belong to another run entry."""

    group: Optional[int] = None
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    writes: bool = True


class Mixer(Part):
    role = "mixer"

    def cache_spec(self) -> Optional[CacheSpec]:
        return None

    def forward(self, x, residual, ctx, cache: Optional[CacheView]) -> None:
        raise NotImplementedError


class FeedForward(Part):
    role = "ffn"

    def forward(self, x, residual, ctx) -> None:
        raise NotImplementedError


class Norm(Part):
    role = "norm"

    def forward(self, residual, ctx):
        raise NotImplementedError

    def forward_rows(self, residual, rows, ctx):
        raise NotImplementedError


class PositionEncoding(Part):
    role = "position"

    def rotary_table(self):
        return None

    def apply(self, q, k, positions):
        return q, k
