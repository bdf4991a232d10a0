"""Dense feed-forward parts."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config import register_part
from ..weights import WeightSpec
from . import linear as L
from .base import FeedForward, LazyNorm


class GatedMLP(FeedForward):
    """SwiGLU: ``h += (silu(x Wg^T) * (x Wu^T)) Wd^T``
    (src/engine/engine_server.cpp:1875-1880, SiLU as src/ops/elementwise.cu:27-33).

    The gate and up matrices are interleaved row by row at load time, so that one contraction
    produces each (gate, up) pair in adjacent columns and the epilogue writes only
    ``silu(gate) * up``; the down projection adds into the residual stream in its epilogue."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, intermediate_size: int, activation: str = "silu",
                 bias: bool = False, names: Optional[Dict[str, str]] = None):
        if activation != "silu":
            raise ValueError(f"the gated feed-forward implements 'silu', not {activation!r}")
        self.prefix, self.hidden_size, self.intermediate_size, self.bias = prefix, hidden_size, intermediate_size, bias
        self.names = {"gate": "gate_proj", "up": "up_proj", "down": "down_proj"}
        self.names.update(names or {})
        self.w_gate_up = self.b_gate_up = self.w_down = self.b_down = None

    def _n(self, which: str, what: str) -> str:
        return f"{self.prefix}.{self.names[which]}.{what}"

    def weight_specs(self) -> List[WeightSpec]:
        D, I = self.hidden_size, self.intermediate_size
        specs = [WeightSpec(self._n("gate", "weight"), (I, D)), WeightSpec(self._n("up", "weight"), (I, D)),
                 WeightSpec(self._n("down", "weight"), (D, I))]
        if self.bias:
            specs += [WeightSpec(self._n("gate", "bias"), (I,)), WeightSpec(self._n("up", "bias"), (I,)),
                      WeightSpec(self._n("down", "bias"), (D,))]
        return specs

    def bind(self, tensors, dtype, device) -> None:
        g, u = tensors[self._n("gate", "weight")], tensors[self._n("up", "weight")]
        wdt = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        I, D = g.shape
        self.w_gate_up = torch.stack([g.to(wdt), u.to(wdt)], dim=1).reshape(2 * I, D).contiguous()
        self.w_down = tensors[self._n("down", "weight")]
        L.reserve_fused_scratch(device, 2 * I)
        if self.bias:
            bg, bu = tensors[self._n("gate", "bias")].float(), tensors[self._n("up", "bias")].float()
            self.b_gate_up = torch.stack([bg, bu], dim=1).reshape(2 * I).contiguous()
            self.b_down = tensors[self._n("down", "bias")].float().contiguous()

    accepts_lazy_norm = True

    def forward(self, x, residual, ctx=None) -> None:
        if isinstance(x, LazyNorm):
            act = L.linear_normed(x, self.w_gate_up, self.b_gate_up, L.SWIGLU)
        else:
            act = L.linear(x, self.w_gate_up, self.b_gate_up, L.SWIGLU)
        L.linear(act, self.w_down, self.b_down, L.RESIDUAL, residual=residual)


register_part("ffn", "gated_mlp", GatedMLP)
