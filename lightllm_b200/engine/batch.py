"""What one step works on: the batch as the caller gives it, and the context the parts see.

The reference's step takes ``ScheduleStep{entries: {request_idx, num_tokens, start_pos,
is_prefill}}`` and finds the token ids in the request's state
(include/lightllm/engine/scheduler.h:53-68, src/engine/engine_server.cpp:808-865).  Here a
step entry carries its token ids, so a replay can feed any tokens, and at most one entry per
request may appear in a step (the reference lets the same request appear twice and then
attends wrongly, engine_server.cpp:1603-1612).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""

    seq_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class Span:
    """One entry as the kernels see it: consecutive positions of one request."""

    seq_id: Hashable
    slot: int          # the request's state slot
    start: int         # position of the first token
    length: int
    row: int           # first row of the batch that belongs to it


class StepContext:
    """Everything a part may read while a step runs.

    Device arrays (int32): ``token_ids``, ``positions`` [T]; ``span_row``, ``span_len``,
    ``span_pos``, ``span_slot`` [S]; per cache group ``slot_mapping[g]`` [T] (cache row of each
    token) and ``block_tables[g]`` [S, max_pages]; ``want_rows`` [R].  ``spans`` is the same
    information on the host."""

    def __init__(self):
        self.T = 0
        self.spans: List[Span] = []
        self.token_ids: torch.Tensor = None
        self.positions: torch.Tensor = None
        self.span_row: torch.Tensor = None
        self.span_len: torch.Tensor = None
        self.span_pos: torch.Tensor = None
        self.span_slot: torch.Tensor = None
        self.iota: torch.Tensor = None           # [S] 0..S-1
        self.zeros: torch.Tensor = None          # [S] zeros
        self.slot_mapping: List[torch.Tensor] = []
        self.block_tables: List[torch.Tensor] = []
        self.want_rows: torch.Tensor = None
        self.num_want = 0
        self.max_pages = 0
        self.page_size = 0
        self.decode_only = False
        self.max_context = 0
        self.dtype: torch.dtype = torch.float32
        self.device: torch.device = None
        self.cache = None
        self.err: Optional[torch.Tensor] = None
        self._tiles: Dict[int, Any] = {}
        self.memo: Dict[Any, Any] = {}          # per-step values that parts share (e.g. rotary tables)

    @property
    def num_spans(self) -> int:
        return len(self.spans)

    def tiles(self, bq: int, min_len: int = 1, max_len: Optional[int] = None):
        """Tiles of ``bq`` query rows, none crossing a span, over the spans whose length lies in
        ``[min_len, max_len]``: ``(tile_span, tile_q0, count)`` as device int32 arrays.  Built once
        per step for each choice."""
        key = (bq, min_len, max_len)
        hit = self._tiles.get(key)
        if hit is not None:
            return hit
        chosen = [(i, s) for i, s in enumerate(self.spans)
                  if s.length >= min_len and (max_len is None or s.length <= max_len)]
        if len(chosen) == len(self.spans) and bq >= max(s.length for s in self.spans):
            hit = (self.iota, self.zeros, len(self.spans))
        elif not chosen:
            hit = (self.iota, self.zeros, 0)
        else:
            ts, tq = [], []
            for i, s in chosen:
                for q0 in range(0, s.length, bq):
                    ts.append(i)
                    tq.append(q0)
            arr = torch.from_numpy(np.asarray([ts, tq], dtype=np.int32)).to(self.device, non_blocking=False)
            hit = (arr[0], arr[1], len(ts))
        self._tiles[key] = hit
        return hit
