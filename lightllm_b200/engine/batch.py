"""What one step works on: the batch as the caller gives it, and the context the parts see.

The reference's step takes ``ScheduleStep{entries: {request_idx, num_tokens, start_pos,
is_prefill}}`` and finds the token ids in the request's state
(include/lightllm/engine/scheduler.h:53-68, src/engine/engine_server.cpp:808-865).  Here a
step entry carries its token ids, so a replay can feed any tokens, and at most one entry per
request may appear in a step (the reference lets the same request appear twice and then
attends wrongly, engine_server.cpp:1603-1612).
"""
from __future__ import annotations

import math
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


# What the tensor-core attention kernel's time is made of, fitted to B200 measurements (14 heads of 64, one prompt of
# 2,048 to 8,192 rows, pieces of 4 to 64 key tiles; the fit is within 6 us of every measurement): microseconds per key
# tile of the busiest block, a fixed cost of the merge kernel if anything is cut, and its cost per partial result and
# head.  Only their ratios matter here.
_TILE_US, _MERGE_US, _PART_US = 2.56, 10.2, 0.026


def _cut(rows, chunk_tiles):
    items, merges, parts = [], [], 0
    for i, q0, ntiles in rows:
        if ntiles <= chunk_tiles + 1:
            items.append((ntiles, i, q0, 0, ntiles, -1))
            continue
        nchunks = -(-ntiles // chunk_tiles)
        merges.append((i, q0, parts, nchunks))
        for c in range(nchunks):
            nk = min(chunk_tiles, ntiles - c * chunk_tiles)
            items.append((nk, i, q0, c * chunk_tiles, nk, parts + c))
        parts += nchunks
    items.sort(key=lambda t: -t[0])
    return items, merges, parts


def _busiest_block(items, heads: int, slots: int) -> float:
    """Key tiles of the block with the most work when the kernel deals the items (times ``heads``, heads fastest) to
    ``slots`` blocks: one item of every round of ``slots`` items, every other round backwards."""
    lengths = np.repeat(np.fromiter((t[0] for t in items), dtype=np.int64, count=len(items)), heads)
    grid = min(len(lengths), max(1, slots))
    idx = np.arange(len(lengths))
    pos = idx % grid
    slot = np.where((idx // grid) % 2 == 0, pos, grid - 1 - pos)
    return float(np.bincount(slot, weights=lengths, minlength=grid).max())


def cut_attention_rows(rows, chunk_tiles=None, heads=1, slots=1):
    """Cuts row tiles ``(span, q0, key tiles)`` into the work items of the tensor-core attention kernel: a tile
    whose key range is longer than ``chunk_tiles`` (+1) becomes pieces of that many key tiles, which leave partial
    results for the merge kernel.  With ``chunk_tiles=None`` the piece length is chosen for the step: a few candidates
    (the share of key tiles that a block gets anyway when all ``heads`` are spread over ``slots`` resident blocks, some
    multiples of it, and no cut at all) are dealt to the blocks as the kernel deals them, and the one with the least
    estimated time wins: the busiest block's tiles plus what the merge of the partial results costs.  (Measured, one
    prompt, 14 heads, 296 blocks: 2,048 rows 41 us with pieces of 7 against 47 uncut; 4,096 rows 88 us uncut against
    101 with pieces of 16; 8,192 rows 279 against 319.)  Returns ``(items, merges, parts)``: items ``(key tiles, span,
    q0, first key tile, key tiles, part or -1)`` longest first, merges ``(span, q0, first part, parts)``, and the
    number of partial results."""
    if chunk_tiles is not None or not rows:
        return _cut(rows, chunk_tiles if chunk_tiles is not None else 1)
    key = (tuple(r[2] for r in rows), heads, slots)
    chunk = _chosen_chunk.get(key)
    if chunk is None:
        longest = max(key[0])
        share = sum(key[0]) * heads / max(1, slots)
        candidates = sorted({min(longest, max(4, math.ceil(share * f))) for f in (0.34, 0.5, 0.75, 1.0, 1.5, 2.0, 3.0)}
                            | {longest})
        best = None
        for c in candidates:
            items, _, parts = _cut(rows, c)
            cost = _TILE_US * _busiest_block(items, heads, slots)
            if parts:
                cost += _MERGE_US + _PART_US * parts * heads
            if best is None or cost < best[0] - 1e-9:
                best = (cost, c)
        chunk = best[1]
        if len(_chosen_chunk) >= 4096:          # steps of ever new shapes: start over rather than grow
            _chosen_chunk.clear()
        _chosen_chunk[key] = chunk
    return _cut(rows, chunk)


_chosen_chunk: Dict[tuple, int] = {}      # the piece length chosen for (the rows' key tiles, heads, slots)


def rows_as_spans(spans: List[Span], bucket: int, max_rows: int):
    """A mixed step described row by row: every token a span of its own (its request's slot, its own position, its own
    row), then the last row repeated until the rows are a multiple of ``bucket`` (at most ``max_rows``).  Returns the
    new spans and, for every span that came in, the span of its first row (the rows keep their order, so a wanted place
    ``w`` of an entry is still row ``first.row + w``)."""
    rows = [Span(s.seq_id, s.slot, s.start + i, 1, s.row + i) for s in spans for i in range(s.length)]
    firsts, at = [], 0
    for s in spans:
        firsts.append(rows[at])
        at += s.length
    T = len(rows)
    padded = min(-(-T // bucket) * bucket, max_rows)
    last = rows[-1]
    rows += [Span(last.seq_id, last.slot, last.start, 1, T + j) for j in range(padded - T)]
    return rows, firsts


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
        self.rowwise = False                    # a mixed step described row by row: several spans may be one request's
        self.select_rows: Optional[torch.Tensor] = None   # row by row: the wanted rows, picked from the logits of all rows
        self.rows_given = 0                     # the tokens that the entries brought (T counts a row-by-row step's padding)
        self.max_context = 0
        self.dtype: torch.dtype = torch.float32
        self.device: torch.device = None
        self.cache = None
        self.err: Optional[torch.Tensor] = None
        self._tiles: Dict[int, Any] = {}
        self.memo: Dict[Any, Any] = {}          # per-step values that parts share (e.g. rotary tables)
        # Index arrays that parts derive from the batch (tiles, work items) travel with the step's other
        # metadata when they are made before it is copied (in the parts' ``prepare``): ``_staging`` is
        # ``[host int32 array, device int32 tensor, next word, end]`` while that is possible.
        self._staging: Optional[list] = None
        self.staged_words = 0
        self.late_uploads = False               # an array was made after the copy and went up on its own
        self.shape_key: List[Any] = []          # what the step's launches depend on beyond its counts

    @property
    def num_spans(self) -> int:
        return len(self.spans)

    def stage(self, arr: np.ndarray) -> torch.Tensor:
        """The int32 array on the device.  Inside ``prepare`` it is written behind the step's metadata
        and shares their one copy; its address then depends only on the sizes staged before it."""
        arr = np.ascontiguousarray(arr, dtype=np.int32)
        st = self._staging
        if st is not None and st[2] + arr.size <= st[3]:
            host, dev, at = st[0], st[1], st[2]
            host[at: at + arr.size] = arr.reshape(-1)
            st[2] = at + arr.size
            self.staged_words += arr.size
            self.shape_key.append(arr.shape)
            return dev[at: at + arr.size].view(arr.shape)
        self.late_uploads = True
        return torch.from_numpy(arr).to(self.device, non_blocking=False)

    def tiles(self, bq: int, min_len: int = 1, max_len: Optional[int] = None, select: Optional[tuple] = None):
        """Tiles of ``bq`` query rows, none crossing a span, over the spans whose length lies in
        ``[min_len, max_len]`` (of the spans ``select`` names by index, if given): ``(tile_span, tile_q0,
        count)`` as device int32 arrays.  Built once per step for each choice."""
        key = (bq, min_len, max_len, select)
        hit = self._tiles.get(key)
        if hit is not None:
            return hit
        chosen = [(i, self.spans[i]) for i in (range(len(self.spans)) if select is None else select)
                  if self.spans[i].length >= min_len and (max_len is None or self.spans[i].length <= max_len)]
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
            arr = self.stage(np.asarray([ts, tq], dtype=np.int32))
            hit = (arr[0], arr[1], len(ts))
        self.shape_key.append(("tiles", key, hit[2]))
        self._tiles[key] = hit
        return hit

    def attention_items(self, min_len: int, window: int, chunk_tiles: Optional[int] = 4, heads: int = 1,
                        slots: int = 1, select: Optional[tuple] = None):
        """Work items of the tensor-core attention kernel for the spans of at least ``min_len`` rows: tiles
        of 128 query rows whose key range (in tiles of 128 keys) is cut into pieces of ``chunk_tiles``, longest
        first, so that a long prompt's last rows do not set the kernel's time.  With ``chunk_tiles=None`` the
        piece is as long as the work allows: the tiles of all ``heads`` spread over ``slots`` resident blocks give
        each block so many tiles anyway, and shorter pieces would only add partial results to merge (see
        :func:`cut_attention_rows`).  ``select`` names the spans by index instead of all of at least ``min_len`` rows.  Returns
        ``(tile_span, tile_q0, count, cut)`` with ``cut`` as ``ops.paged_attention_tcgen05`` takes it."""
        key = ("items", min_len, window, chunk_tiles, heads, slots, select)
        hit = self._tiles.get(key)
        if hit is not None:
            return hit
        # the row tiles (span, first row, key tiles) of the spans that take part
        rows = []
        for i in (range(len(self.spans)) if select is None else select):
            s = self.spans[i]
            if s.length < min_len:
                continue
            for q0 in range(0, s.length, 128):
                pos0 = s.start + q0
                hi = pos0 + 128 if q0 + 128 <= s.length else s.start + s.length
                lo = pos0 - window + 1 if window > 0 and pos0 >= window else 0
                rows.append((i, q0, -(-(hi - (lo // 128) * 128) // 128)))
        items, merges, parts = cut_attention_rows(rows, chunk_tiles, heads, slots)
        if not items:
            hit = (self.iota, self.zeros, 0, None)
        else:
            arr = self.stage(np.asarray([t[1:] for t in items], dtype=np.int32).T)
            self.shape_key.append(("parts", parts))
            cut = None
            if merges:
                m = self.stage(np.asarray(merges, dtype=np.int32).T)
                cut = (arr[2], arr[3], arr[4], parts, m[0], m[1], m[2], m[3], len(merges))
            else:
                cut = (arr[2], arr[3], arr[4], 0, None, None, None, None, 0)
            hit = (arr[0], arr[1], len(items), cut)
        self._tiles[key] = hit
        return hit
