"""RMSNorm of the float32 residual stream."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config import register_part
from ..csrc import ops
from ..weights import WeightSpec
from .base import Norm


class RMSNorm(Norm):
    """``y = x / sqrt(mean(x^2) + eps) * weight`` with the statistics in float32
    (src/ops/norm.cu:19-23,48-54).  ``weight_name`` is the full checkpoint name."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, eps: float, weight_name: str = "weight"):
        self.name = f"{prefix}.{weight_name}" if prefix else weight_name
        self.hidden_size = hidden_size
        self.eps = float(eps)
        self.weight = None
        self.out_dtype = torch.float32

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.name, (self.hidden_size,), init=("one_plus_normal", 0.01))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weight = tensors[self.name]
        self.out_dtype = dtype

    def rms_parameters(self):
        """(weight, eps) for kernels that fold this norm into their prologue."""
        return self.weight, self.eps

    def forward(self, residual, ctx=None):
        out = torch.empty(residual.shape, dtype=self.out_dtype, device=residual.device)
        ops.rmsnorm(residual, self.weight, self.eps, out)
        return out

    def forward_rows(self, residual, rows, ctx=None):
        out = torch.empty((rows.numel(), self.hidden_size), dtype=self.out_dtype, device=residual.device)
        ops.rmsnorm(residual, self.weight, self.eps, out, rows=rows)
        return out


register_part("norm", "rmsnorm", RMSNorm)
