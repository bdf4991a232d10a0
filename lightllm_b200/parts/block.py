"""A block: two norms, a mixer and a feed-forward in a given arrangement."""
from __future__ import annotations

from typing import List

from ..config import LayerSpec, part_class
from .base import LazyNorm, Part

ARRANGEMENTS = ("pre_norm", "parallel")


def build_part(role: str, spec):
    return part_class(role, spec.kind)(spec.prefix, **spec.params)


class Block(Part):
    """``pre_norm``:  h += mixer(norm1(h)); h += ffn(norm2(h))   (src/engine/engine_server.cpp:1530-1880)
    ``parallel``:  both branches read the same h, then both are added."""

    role = "block"

    def __init__(self, spec: LayerSpec):
        if spec.arrangement not in ARRANGEMENTS:
            raise ValueError(f"unknown arrangement {spec.arrangement!r}; known: {ARRANGEMENTS}")
        self.arrangement = spec.arrangement
        self.norm1 = build_part("norm", spec.norm1)
        self.mixer = build_part("mixer", spec.mixer)
        self.norm2 = build_part("norm", spec.norm2)
        self.ffn = build_part("ffn", spec.ffn)

    def children(self) -> List[Part]:
        return [self.norm1, self.mixer, self.norm2, self.ffn]

    @staticmethod
    def _normed(part, norm, residual, ctx):
        """The part's input: the norm left to the part when it can fold it into its first kernel."""
        if part.accepts_lazy_norm:
            return LazyNorm(residual, norm, ctx)
        return norm.forward(residual, ctx)

    def prepare(self, ctx, cache=None) -> None:
        for part in (self.norm1, self.norm2, self.ffn):
            hook = getattr(part, "prepare", None)
            if hook is not None:
                hook(ctx)
        hook = getattr(self.mixer, "prepare", None)
        if hook is not None:
            hook(ctx, cache)

    def forward(self, residual, ctx, cache) -> None:
        if self.arrangement == "pre_norm":
            self.mixer.forward(self._normed(self.mixer, self.norm1, residual, ctx), residual, ctx, cache)
            self.ffn.forward(self._normed(self.ffn, self.norm2, residual, ctx), residual, ctx)
        else:   # both branches read the same h, so both norms are computed before anything is added
            x1 = self.norm1.forward(residual, ctx)
            x2 = self.norm2.forward(residual, ctx)
            self.mixer.forward(x1, residual, ctx, cache)
            self.ffn.forward(x2, residual, ctx)
