"""A block: two norms, a mixer and a feed-forward in a given arrangement."""
from __future__ import annotations

from typing import List

from ..config import LayerSpec, part_class
from .base import Part

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

    def forward(self, residual, ctx, cache) -> None:
        if self.arrangement == "pre_norm":
            self.mixer.forward(self.norm1.forward(residual, ctx), residual, ctx, cache)
            self.ffn.forward(self.norm2.forward(residual, ctx), residual, ctx)
        else:
            x1 = self.norm1.forward(residual, ctx)
            x2 = self.norm2.forward(residual, ctx)
            self.mixer.forward(x1, residual, ctx, cache)
            self.ffn.forward(x2, residual, ctx)
