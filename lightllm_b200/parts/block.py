"""A block: sub-blocks (norm before, a mixer or feed-forward, norm after) around the residual stream."""
from __future__ import annotations

from typing import List, Optional

import torch

from ..config import LayerSpec, part_class
from ..csrc import ops
from .base import LazyNorm, Part


def build_part(role: str, spec):
    return part_class(role, spec.kind)(spec.prefix, **spec.params)


class BuiltSubBlock:
    """The parts of one :class:`~lightllm_b200.config.SubBlock`."""

    def __init__(self, spec):
        self.role = spec.role
        self.part = build_part(spec.role, spec.part)
        self.norm_before = build_part("norm", spec.norm_before) if spec.norm_before is not None else None
        self.norm_after = build_part("norm", spec.norm_after) if spec.norm_after is not None else None
        self.after = spec.after

    def parts(self) -> List[Part]:
        return [p for p in (self.norm_before, self.part, self.norm_after) if p is not None]


class Block(Part):
    """``sequential``: every sub-block reads the stream the one before it left, e.g. Qwen2's
    ``h += mixer(norm1(h)); h += ffn(norm2(h))`` (src/engine/engine_server.cpp:1530-1880);
    ``parallel``: all sub-blocks read the same h, then every branch is added.
    What a sub-block may hold is described at :class:`~lightllm_b200.config.SubBlock`."""

    role = "block"

    def __init__(self, spec: LayerSpec):
        self.arrangement = spec.arrangement
        self.subs: List[BuiltSubBlock] = [BuiltSubBlock(sb) for sb in spec.sub_blocks]
        mixers = [sb.part for sb in self.subs if sb.role == "mixer"]
        self.mixer: Optional[Part] = mixers[0] if mixers else None

    def children(self) -> List[Part]:
        return [p for sb in self.subs for p in sb.parts()]

    @staticmethod
    def _input(sb: BuiltSubBlock, residual, ctx, lazy: bool):
        """The part's input: the norm left to the part when it can fold it into its first kernel."""
        if sb.norm_before is None:
            dtype = ctx.dtype if ctx is not None and ctx.dtype is not None else residual.dtype
            if dtype == residual.dtype:
                return residual
            x = torch.empty(residual.shape, dtype=dtype, device=residual.device)
            ops.cast_add(residual, x)
            return x
        if lazy and sb.part.accepts_lazy_norm:
            return LazyNorm(residual, sb.norm_before, ctx)
        return sb.norm_before.forward(residual, ctx)

    @staticmethod
    def _run(sb: BuiltSubBlock, x, residual, ctx, cache) -> None:
        branch = sb.norm_after is not None and sb.after == "branch"
        target = residual
        if branch:      # the part adds into a cleared buffer, which is normed and then added to the stream
            target = torch.zeros_like(residual)
        elif x is residual:      # a part without a norm before it, in float32: it must not read what it adds into
            x = residual.clone()
        if sb.role == "mixer":
            sb.part.forward(x, target, ctx, cache)
        else:
            sb.part.forward(x, target, ctx)
        if branch:
            ops.cast_add(sb.norm_after.forward(target, ctx), residual, accumulate=True)
        elif sb.norm_after is not None:
            ops.cast_add(sb.norm_after.forward(residual, ctx), residual)

    def forward(self, residual, ctx, cache) -> None:
        if self.arrangement == "parallel":
            # every branch reads the same h, so all inputs are computed before anything is added
            inputs = [self._input(sb, residual, ctx, lazy=False) for sb in self.subs]
            inputs = [x.clone() if x is residual else x for x in inputs]
            for sb, x in zip(self.subs, inputs):
                self._run(sb, x, residual, ctx, cache)
        else:
            for sb in self.subs:
                self._run(sb, self._input(sb, residual, ctx, lazy=True), residual, ctx, cache)
