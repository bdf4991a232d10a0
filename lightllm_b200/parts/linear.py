"""The dense contraction every part uses, with its fused epilogues.

``y = x @ W^T`` with ``W`` stored ``[out, in]`` as in the checkpoint
(src/engine/engine_server.cpp:1542-1544).  Which kernel runs depends on dtype and shape only:

* float32 activations: the CUDA-core FFMA kernels (true 32-bit, no tensor cores);
* bfloat16 activations and weights, rows of 16-byte multiples, more than a few rows:
  the tcgen05 tensor-core kernel with TMEM accumulators;
* everything else (few rows, odd inner sizes, float32 weights under bfloat16 activations):
  the CUDA-core kernels, which take any size.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops

STORE, STORE_F32, RESIDUAL, SWIGLU = ops.EPI_STORE, ops.EPI_STORE_F32, ops.EPI_RESIDUAL, ops.EPI_SWIGLU

# Rows at or below which the row-streaming CUDA-core kernel is used for bfloat16 (decode).
SMALL_M = 0
NUM_SMS = 148


def tensor_core_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and M > SMALL_M
            and ops.has_tcgen05())


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, epilogue: int = STORE,
           out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None) -> Optional[torch.Tensor]:
    """Run the contraction; returns ``out`` (allocated here when not given), or ``None`` for the
    residual epilogue, which adds into ``residual``."""
    M, N = x.shape[0], w.shape[0]
    if epilogue != RESIDUAL and out is None:
        cols = N // 2 if epilogue == SWIGLU else N
        dt = torch.float32 if epilogue == STORE_F32 else x.dtype
        out = torch.empty((M, cols), dtype=dt, device=x.device)
    if M == 0:
        return out
    if tensor_core_eligible(x, w):
        split_k = 1
        if epilogue == RESIDUAL and M <= 128:
            # few rows: the grid has only N/128 blocks; cut K so that the weights stream from all SMs
            tiles, kblocks = -(-N // 128), -(-x.shape[1] // 64)
            split_k = max(1, min(kblocks, NUM_SMS // tiles))
        ops.gemm_tcgen05(x, w, bias, epilogue, out, residual, split_k)
    else:
        ops.gemm_simt(x, w, bias, epilogue, out, residual)
    return out
