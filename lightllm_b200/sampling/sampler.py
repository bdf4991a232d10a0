"""Choosing the next token of every row of logits, on the device.

The reference copies each row of logits to the host and samples there
(src/engine/engine_server.cpp:2043-2051, src/ops/sampling.cpp:22-335).  Here the rows stay on
the device: greedy rows go through the argmax kernel, the rest through the sampling kernel
(temperature, top-k, top-p, min-p and the draw); only the chosen ids come back.  The uniform
number of each draw comes from the request's own counter-based stream (Philox keyed by the
request's seed and id), so a request's output does not depend on what else is in the batch.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Sequence

import numpy as np
import torch

from ..csrc import ops
from .params import SamplingParams


class RequestStream:
    """The random stream of one request: draw ``n`` gives the same number whatever happened to
    other requests."""

    def __init__(self, seed: int, request_id: int):
        key = (int(seed) & 0xFFFF_FFFF_FFFF_FFFF, int(request_id) & 0xFFFF_FFFF_FFFF_FFFF)
        self._gen = np.random.Generator(np.random.Philox(key=np.array(key, dtype=np.uint64)))

    def uniform(self) -> float:
        return float(self._gen.random(dtype=np.float32))


class Sampler:
    def __init__(self, device: torch.device):
        self.device = device
        self._streams: Dict[Hashable, RequestStream] = {}

    def stream(self, request_id: int, seed: int) -> RequestStream:
        s = self._streams.get(request_id)
        if s is None:
            s = self._streams[request_id] = RequestStream(seed, request_id)
        return s

    def forget(self, request_id: int) -> None:
        self._streams.pop(request_id, None)

    def sample(self, logits: torch.Tensor, request_ids: Sequence[int], params: Sequence[SamplingParams]) -> List[int]:
        """One token id per row of ``logits`` (float32 ``[R, V]`` on the device)."""
        tokens = self.sample_device(logits, request_ids, params)
        return tokens.cpu().tolist()

    def sample_device(self, logits: torch.Tensor, request_ids: Sequence[int],
                      params: Sequence[SamplingParams]) -> torch.Tensor:
        R = logits.shape[0]
        if len(request_ids) != R or len(params) != R:
            raise ValueError(f"{R} rows of logits but {len(request_ids)} requests and {len(params)} parameter sets")
        out = torch.empty(R, dtype=torch.int32, device=logits.device)
        if all(p.greedy for p in params):
            ops.argmax(logits, out)
            return out
        host = np.zeros((5, R), dtype=np.float32)
        for i, (rid, p) in enumerate(zip(request_ids, params)):
            host[0, i], host[1, i], host[2, i] = p.temperature, p.top_p, p.min_p
            host[3, i] = 0.0 if p.greedy else self.stream(rid, p.seed).uniform()
            host[4, i] = np.int32(p.top_k).view(np.float32)
        dev = torch.from_numpy(host).to(logits.device)
        ops.sample(logits, dev[0], dev[4].view(torch.int32), dev[1], dev[2], dev[3], out)
        return out
