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
_num_sms = {}


def num_sms(device=None) -> int:
    """Multiprocessors of the device the step runs on (asked once)."""
    idx = torch.cuda.current_device() if device is None else (torch.device(device).index or 0)
    n = _num_sms.get(idx)
    if n is None:
        n = _num_sms[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return n


def tensor_core_eligible(x: torch.Tensor, w: torch.Tensor) -> bool:
    M, K = x.shape
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0 and M > SMALL_M
            and ops.has_tcgen05())


DECODE_ROWS = 64     # steps of at most this many rows use the fused decode contraction
# Rows up to which the norm is folded into the contraction's prologue.  Measured on B200 at Qwen2.5-0.5B sizes the
# separate norm kernel wins at every size: at 8 rows the prologue (each block reads the rows, one trip to memory
# before its first MMA) makes gate/up 10.2 us against 7.5 + 1.7, and the decode step 0.95 ms against 0.89.  So it is
# off; the prologue stays built and tested.
FUSE_NORM_MAX_ROWS = 0
FUSE_NORM_MAX_COLS = 1024


def decode_eligible(M: int, w: torch.Tensor, act_dtype: torch.dtype, norm: bool, epilogue: int, head_dim: int = 0) -> bool:
    return (M <= DECODE_ROWS and act_dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and ops.has_tcgen05()
            and ops.gemm_decode_supports(M, w.shape[0], w.shape[1], norm, epilogue, head_dim))


def split_k_for(M: int, N: int, K: int) -> int:
    """Few rows leave only N/128 blocks; cut K so that the weights stream from all SMs."""
    tiles, kblocks = -(-N // 128), -(-K // 64)
    return max(1, min(kblocks, num_sms() // tiles))


def split_k_fused(M: int, N: int, K: int) -> int:
    """Splits for a decode contraction whose epilogue is fused (the splits meet in scratch).  Meeting
    costs three more round trips to memory, so it only pays when the grid would otherwise leave most
    SMs idle (the q/k/v projection: 9 blocks), and only for few rows, where the atomic adds are cheap."""
    tiles, kblocks = -(-N // 128), -(-K // 64)
    if M > 16 or tiles * 4 > num_sms():
        return 1
    return max(1, min(kblocks, num_sms() // tiles))


def split_k_wide(M: int, N: int, K: int) -> int:
    """Splits for a contraction of more than 128 rows.  A block's time is its number of tensor-core
    instructions (K/16 per tile, whatever the tile's width), so when the tiles of 128 rows x 256 features
    leave half of the SMs idle, K is cut until they do not.  The pieces meet through memory, which costs about
    as much as 16 blocks of 64 along K: shorter pieces do not pay."""
    tiles = -(-M // 128) * -(-N // (256 if N > 128 else 128))
    if tiles * 2 > num_sms():
        return 1
    return max(1, min(num_sms() // tiles, -(-K // 64) // 16))


def reserve_fused_scratch(device: torch.device, N: int) -> None:
    """Called when a part with a fused decode contraction of N output features is bound."""
    if torch.device(device).type == "cuda":
        ops.reserve_splitk_scratch(device, DECODE_ROWS * N, -(-N // 128))


_DECODE_EPI = {STORE_F32: ops.DEPI_STORE_F32, RESIDUAL: ops.DEPI_RESIDUAL, SWIGLU: ops.DEPI_SWIGLU}


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

    if epilogue in _DECODE_EPI and decode_eligible(M, w, x.dtype, False, _DECODE_EPI[epilogue]):
        split_k = 1
        if epilogue == RESIDUAL:
            split_k = split_k_for(M, N, x.shape[1])
        elif epilogue == SWIGLU:
            split_k = split_k_fused(M, N, x.shape[1])
        ops.gemm_decode(w, _DECODE_EPI[epilogue], M, a=x, bias=bias, out=out, residual=residual, split_k=split_k)
    elif tensor_core_eligible(x, w):
        if M > 128:
            split_k = split_k_wide(M, N, x.shape[1])
        else:
            split_k = split_k_for(M, N, x.shape[1]) if epilogue == RESIDUAL else 1
        ops.gemm_tcgen05(x, w, bias, epilogue, out, residual, split_k)
    else:
        ops.gemm_simt(x, w, bias, epilogue, out, residual)
    return out


def linear_normed(lazy, w: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int) -> torch.Tensor:
    """``linear`` on a LazyNorm input: the norm runs inside the contraction when the shape allows."""
    M, N = lazy.num_rows, w.shape[0]
    rms = lazy.fusable()
    if rms is not None and epilogue in _DECODE_EPI and 0 < M <= FUSE_NORM_MAX_ROWS and w.shape[1] <= FUSE_NORM_MAX_COLS and \
            decode_eligible(M, w, lazy.norm.out_dtype, True, _DECODE_EPI[epilogue]):
        cols = N // 2 if epilogue == SWIGLU else N
        out = torch.empty((M, cols), dtype=torch.float32 if epilogue == STORE_F32 else torch.bfloat16,
                          device=w.device)
        ops.gemm_decode(w, _DECODE_EPI[epilogue], M, x=lazy.residual, x_rows=lazy.rows, norm_weight=rms[0],
                        eps=rms[1], bias=bias, out=out,
                        split_k=split_k_fused(M, N, w.shape[1]) if epilogue == SWIGLU else 1)
        return out
    return linear(lazy.materialize(), w, bias, epilogue)
