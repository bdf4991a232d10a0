"""The step function: one batch of (request, its next tokens) in, logits at the wanted places out.

It runs only the tokens it is given, as one batch, against the cache that earlier steps left:
portions of prompts beside single decoded tokens, cut anywhere.  The reference's
``EngineServer::step`` (src/engine/engine_server.cpp:1350-2123) splits its entries into three
attention paths (:1603-1612), re-uploads block tables for every layer (:1793-1809),
synchronises the device per layer (:1589) and samples inside the step; here there is one path,
one host-to-device copy of the step's metadata, no synchronisation, and the step returns logits
(sampling is the caller's).
"""
from __future__ import annotations

import logging
import os
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache import CacheManager
from ..csrc import ops
from ..models import Model
from ..parts import CacheView
from ..parts.base import LazyNorm
from .batch import Span, StepContext, StepEntry, rows_as_spans
from .fused_decode import FusedDecode
from .native_step import NativeLayers


class StepError(ValueError):
    """The batch given to a step is malformed."""


class ModelRunner:
    """Owns the device-side step metadata and runs the model over a batch."""

    # A mixed step's shape is captured into a graph when it comes for this many-th time.
    MIXED_CAPTURE_AFTER = 6
    # A step of few rows that mixes portions and decoded tokens is described to the kernels row by row: every token a
    # span of its own (its request's block table, its own position).  The keys and values of all rows are in the cache
    # before any row's attention reads them, and a row sees the positions up to its own, so the logits are the same;
    # but the step now has the shape of a decoding batch of as many rows, whatever its composition: it takes the decode
    # kernels launched one after the other (not the persistent layer kernel, whose attention stage makes a row's new key
    # and value itself and so wants one row a request), needs no work items cut for it on the host, and its shape, which
    # depends on its counts alone, comes again for a CUDA graph.  Measured at the 0.5B sizes (a 16-token portion beside 1
    # to 16 decoded tokens, contexts of 300 to 4,000; bench.py --only small-mixed): 1.65 ms a step with the portion kept
    # whole, 1.17 ms row by row.
    # Each row reads its keys by itself, so the rule holds only while the portions' rows x keys stay small.
    # Such a step is padded to a multiple of ROWWISE_BUCKET rows by repeating its last row (the same token at the same
    # position writes the same key and value to the same place, and its output is dropped), and its logits are computed
    # for every row and the wanted ones picked afterwards: then its shape, and its graph, depend on nothing but the
    # bucket and the block-table width, and nearly every such step is a replay.
    ROWWISE_MAX_ROWS = 64
    ROWWISE_MAX_ROW_KEYS = 1 << 17
    ROWWISE_BUCKET = 8

    def __init__(self, model: Model, cache: CacheManager, max_batch_tokens: int, max_spans: Optional[int] = None,
                 use_cuda_graphs: bool = True, max_graphs: int = 64):
        if model.device is None or model.device.type != "cuda":
            raise RuntimeError("the model is not on a CUDA device; the engine has no CPU path")
        self.model = model
        self.cache = cache
        self.device = model.device
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_spans = int(max_spans or cache.max_seqs)
        self.ngroups = len(cache.layout.groups)
        self.max_pages = cache.max_pages_per_seq
        # Capacity of the metadata buffer (int32 words).  A step packs its arrays tightly at
        # offsets that depend only on its counts, so equal counts give equal addresses.
        S, T, G, P = (max(self.max_spans, self.ROWWISE_MAX_ROWS), max(self.max_batch_tokens, self.ROWWISE_MAX_ROWS),
                      self.ngroups, self.max_pages)
        self._map_cap = S                    # rows of a step that may take their ids from the device (token_map)
        off = 2 * self._map_cap + 6 * S + G * S * P + T + 2 * T + G * T
        self._fixed_words = off
        off += 8 * T + 64 * S + 4096         # room for the index arrays that parts stage (tiles, work items)
        self._words = off
        self._host = [torch.zeros(off, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._host_done = [None, None]
        self._turn = 0
        self._dev = torch.zeros(off, dtype=torch.int32, device=self.device)
        self.err = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.views: List[Optional[CacheView]] = []
        for ref in cache.layout.refs:
            if ref.group is None and ref.state_plane is None:
                self.views.append(None)
                continue
            k = v = None
            if ref.group is not None:
                k, v = cache.plane_kv(ref.group, ref.plane)
            st = cache.state[ref.state_plane] if ref.state_plane is not None else None
            self.views.append(CacheView(ref.group, k, v, st, ref.owns))
        self.last_h2d_bytes = 0
        self.last_ctx: Optional[StepContext] = None
        self._nvtx = os.environ.get("LLB_NVTX", "") not in ("", "0")
        # Steps are launch-bound on the host, so they are captured into CUDA graphs: one per shape (counts of
        # tokens, requests, wanted rows, block-table width, sizes of the staged index arrays), captured the
        # second time a shape is seen.
        self.graph_blockers = model.graph_blockers()      # the parts (by class name) that keep steps out of graphs
        self.use_cuda_graphs = bool(use_cuda_graphs) and not self.graph_blockers
        if use_cuda_graphs and self.graph_blockers:
            logging.getLogger("lightllm_b200").info(
                "steps run launch by launch, not from CUDA graphs: %s do(es) not declare graph_safe",
                ", ".join(self.graph_blockers))
        self.max_graphs = max_graphs
        self._graphs: Dict[tuple, tuple] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_pool = None
        self._capture_stream = None
        self.graph_replays = 0
        self.graph_launches = 0          # kernels launched through graph replays
        # Decode steps run the common layers as one persistent kernel per segment of the run list.
        self.fused = FusedDecode(model, self.views, self.device)
        # Every other step runs them through the library's step executor: one call for a stretch of run entries.
        self.native = NativeLayers(model, self.views, self.device)
        # Row-by-row steps need every run entry to be the common attention block (a part with state of its own keeps one
        # state per request, not per row): exactly the entries that the step executor covers.
        self.rowwise = (os.environ.get("LLB_ROWWISE_STEPS", "1") not in ("0", "") and self.native.enabled
                        and len(self.native.covers) > 0 and all(self.native.covers))

    # ------------------------------------------------------------------------------------------
    def _build_context(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None,
                       token_map=None) -> StepContext:
        cache = self.cache
        vocab = self.model.spec.vocab_size
        if not entries:
            raise StepError("a step needs at least one entry")
        if len(entries) > self.max_spans:
            raise StepError(f"{len(entries)} entries in one step; the limit is {self.max_spans}")
        seen = set()
        spans: List[Span] = []
        row = 0
        for e in entries:
            if e.seq_id in seen:
                raise StepError(f"request {e.seq_id!r} appears twice in one step")
            seen.add(e.seq_id)
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.seq_id!r} brings no tokens")
            seq = cache.get(e.seq_id)
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.seq_id!r} wants place {w} of {n} tokens")
            spans.append(Span(e.seq_id, seq.slot, seq.length, n, row))
            row += n
        T = row
        if T > self.max_batch_tokens:
            raise StepError(f"{T} tokens in one step; the limit is {self.max_batch_tokens}")
        if max(s.start + s.length for s in spans) > self.model.spec.max_positions:
            raise StepError(f"a request would pass the model's {self.model.spec.max_positions} positions")

        max_context = max(s.start + s.length for s in spans)
        # (what the rows of portions read beyond what the portions kept whole would: each row its keys by itself)
        portion_keys = sum(s.length * (s.start + s.length) for s in spans if s.length > 1)
        if self.rowwise and T <= self.ROWWISE_MAX_ROWS and 0 < portion_keys <= self.ROWWISE_MAX_ROW_KEYS:
            spans, span_of_entry = rows_as_spans(spans, self.ROWWISE_BUCKET, self.ROWWISE_MAX_ROWS)
            rowwise = True
        else:
            span_of_entry, rowwise = spans, False
        real_T, T = T, len(spans) if rowwise else T
        S, G = len(spans), self.ngroups
        if len(entries) == 1:
            ids = np.asarray(entries[0].tokens, dtype=np.int64)
        else:
            ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        if ids.min() < 0 or ids.max() >= vocab:
            bad = int(ids[(ids < 0) | (ids >= vocab)][0])
            raise StepError(f"token id {bad} is outside the vocabulary of {vocab}")
        if T > real_T:
            ids = np.concatenate([ids, np.full(T - real_T, ids[-1], dtype=np.int64)])
        # Pages for the new tokens are taken before anything runs; OutOfPages leaves all as it was.
        cache.reserve_all((e.seq_id, len(e.tokens)) for e in entries)

        ps = cache.page_size
        # Block-table width of this step: the pages of its longest request, rounded up to 32, so that a
        # decoding batch keeps its shape (and its captured graph) for hundreds of steps.
        P = min(self.max_pages, -(-(-(-max_context // ps)) // 32) * 32)
        want = [s.row + w for s, e in zip(span_of_entry, entries) for w in e.want]
        R = len(want)
        want_words = T if rowwise else R          # row by row: a field of the bucket's size, whatever is wanted
        o, off = {}, 0
        # token_map: (ids on the device, rows of this step, places in those ids): these rows take their ids from there
        # (the ids a step in flight is sampling).  Padding rows that repeat such a row repeat its id.
        map_rows: List[int] = []
        map_from: List[int] = []
        if token_map is not None:
            map_rows, map_from = list(token_map[1]), list(token_map[2])
            if map_rows and T > real_T and map_rows[-1] == real_T - 1:
                map_rows += list(range(real_T, T))
                map_from += [map_from[-1]] * (T - real_T)
        K = len(map_rows)
        if K > self._map_cap:
            raise StepError(f"{K} rows take their ids from the device; the limit is {self._map_cap}")
        # The two lists of the map have a place of fixed size at the head of the buffer: no other array's place may depend
        # on how many rows the map names, since a CUDA graph captured for this shape reads those arrays where they lay then.
        fields = (("map_rows", self._map_cap), ("map_from", self._map_cap),
                  ("span_row", S), ("span_len", S), ("span_pos", S), ("span_slot", S), ("iota", S),
                  ("zeros", S), ("block_tables", G * S * P), ("want_rows", want_words), ("token_ids", T),
                  ("positions", T), ("slot_mapping", G * T))
        for name, n in fields:
            o[name] = off
            off += n
        words = off

        turn = self._turn
        self._turn ^= 1
        if self._host_done[turn] is not None:
            self._host_done[turn].synchronize()
        host = self._host[turn].numpy()
        host[o["token_ids"]: o["token_ids"] + T] = ids
        if S == 1:
            pos = np.arange(spans[0].start, spans[0].start + T, dtype=np.int32)
        elif S == T:
            pos = np.fromiter((s.start for s in spans), dtype=np.int32, count=T)
        else:
            pos = np.concatenate([np.arange(s.start, s.start + s.length, dtype=np.int32) for s in spans])
        host[o["positions"]: o["positions"] + T] = pos
        host[o["span_row"]: o["span_row"] + S] = [s.row for s in spans]
        host[o["span_len"]: o["span_len"] + S] = [s.length for s in spans]
        host[o["span_pos"]: o["span_pos"] + S] = [s.start for s in spans]
        host[o["span_slot"]: o["span_slot"] + S] = [s.slot for s in spans]
        host[o["iota"]: o["iota"] + S] = np.arange(S, dtype=np.int32)
        host[o["zeros"]: o["zeros"] + S] = 0
        for g in range(G):
            bt = host[o["block_tables"] + g * S * P: o["block_tables"] + (g + 1) * S * P].reshape(S, P)
            sm = host[o["slot_mapping"] + g * T: o["slot_mapping"] + (g + 1) * T]
            tables_of = {}
            for i, s in enumerate(spans):
                table = tables_of.get(s.seq_id)
                if table is None:
                    table = tables_of[s.seq_id] = cache.block_table_array(s.seq_id, g)
                bt[i, : len(table)] = table[:P]
                bt[i, len(table):] = -1          # "no page": what an earlier step left in the buffer is never an id
                p = pos[s.row: s.row + s.length]
                rows = table[p // ps]
                if rows.min() < 0:
                    raise StepError(f"request {s.seq_id!r}: a new token falls in a page that was given back")
                sm[s.row: s.row + s.length] = rows * ps + p % ps
        host[o["want_rows"]: o["want_rows"] + R] = want
        if K:
            if min(map_rows) < 0 or max(map_rows) >= T or min(map_from) < 0 or max(map_from) >= token_map[0].numel():
                raise StepError("the map of device token ids names a row or a place that does not exist")
            host[o["map_rows"]: o["map_rows"] + K] = map_rows
            host[o["map_from"]: o["map_from"] + K] = map_from

        d = self._dev
        ctx = StepContext()
        ctx.T, ctx.spans = T, spans
        # one view per field, cut in one call (a slice each costs the host a microsecond or more)
        (map_rows_dev, map_from_dev, ctx.span_row, ctx.span_len, ctx.span_pos, ctx.span_slot, ctx.iota, ctx.zeros, tables,
         ctx.want_rows, ctx.token_ids, ctx.positions, slots) = d[:words].split_with_sizes([n for _, n in fields])
        if G == 1:
            ctx.slot_mapping, ctx.block_tables = [slots], [tables.view(S, P)]
        else:
            ctx.slot_mapping = list(slots.split(T))
            ctx.block_tables = [t.view(S, P) for t in tables.split(S * P)]
        ctx.num_want = R
        ctx.select_rows = None
        if rowwise:
            # the head runs over every row of the bucket; the wanted rows are picked from its result
            ctx.select_rows = ctx.want_rows[:R]
            ctx.want_rows = ctx.iota
            ctx.num_want = T if R else 0
        ctx.rows_given = real_T
        ctx.max_pages, ctx.page_size = P, ps
        ctx.decode_only = all(s.length == 1 for s in spans)
        ctx.rowwise = rowwise
        ctx.max_context = max_context
        ctx.dtype, ctx.device = self.model.dtype, self.device
        ctx.cache, ctx.err = cache, self.err

        # The parts make their index arrays now, behind the fixed fields, so that one copy brings everything.
        ctx._staging = [host, d, words, self._words]
        self.model.prepare(ctx, self.views)
        words = ctx._staging[2]
        ctx._staging = None
        self._dev[:words].copy_(self._host[turn][:words], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record(ops.torch_stream())
        self._host_done[turn] = ev
        self.last_h2d_bytes = words * 4
        if device_tokens is not None:
            # the tokens of this step are still on the device (the ids the last step sampled)
            if device_tokens.dtype != torch.int32 or device_tokens.numel() != real_T or not device_tokens.is_cuda:
                raise StepError(f"device tokens must be {real_T} int32 values on the device")
            ctx.token_ids[:real_T].copy_(device_tokens.reshape(-1))
            if T > real_T:           # the padding repeats the last row, so it must bring the last row's token
                ctx.token_ids[real_T:].copy_(device_tokens.reshape(-1)[-1:].expand(T - real_T))
        if K:
            src = token_map[0]
            if src.dtype != torch.int32 or not src.is_cuda:
                raise StepError("mapped device tokens must be int32 values on the device")
            ctx.token_ids[map_rows_dev[:K]] = src.reshape(-1).index_select(0, map_from_dev[:K])
        return ctx

    def forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Run the layers over the batch that ``ctx`` describes; logits float32 [R, V] or None.
        With ``LLB_NVTX=1`` in the environment every run entry is an NVTX range (the reference only has
        ``printf`` timings, src/engine/batch_loop.cpp:99-102)."""
        from ..csrc import ops
        with ops.stream_scope():           # every kernel of the step goes to the stream that is current now
            return self._forward(ctx)

    def _forward(self, ctx: StepContext) -> Optional[torch.Tensor]:
        m = self.model
        residual = m.embedding.forward(ctx.token_ids, ctx)
        fused = self.fused if self.fused.takes(ctx) else None
        i = 0
        while i < len(m.run):
            segment = fused.segment_at(i) if fused is not None else None
            if self._nvtx:
                torch.cuda.nvtx.range_push(f"run{i}:" + (f"fused to {segment.end}" if segment else f"layer{m.run[i].layer}"))
            if segment is not None:
                segment.run(residual, ctx)
                i = segment.end
            elif self.native.covers[i]:
                j = self.native.stretch(i)
                if fused is not None:           # up to where the next fused segment begins
                    j = next((k for k in range(i + 1, j) if fused.segment_at(k) is not None), j)
                self.native.run(residual, ctx, i, j)
                i = j
            else:
                m.layers[m.run[i].layer].forward(residual, ctx, self.views[i])
                i += 1
            if self._nvtx:
                torch.cuda.nvtx.range_pop()
        if ctx.num_want == 0:
            return None
        if m.head.accepts_lazy_norm:
            return m.head.forward(LazyNorm(residual, m.final_norm, ctx, rows=ctx.want_rows), ctx)
        return m.head.forward(m.final_norm.forward_rows(residual, ctx.want_rows, ctx), ctx)

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None,
             token_map=None) -> Optional[torch.Tensor]:
        """One step.  Returns the logits at the wanted places, in the order of the entries and of
        each entry's ``want``, as a float32 ``[wanted, vocab]`` tensor on the device (``None`` if
        nothing is wanted).  Afterwards every request holds its new tokens.  With ``device_tokens`` (int32,
        one per token of the step, on the device) the entries' own token ids only give the counts: the step
        reads its ids from that tensor, so ids that were sampled on the device need not visit the host.
        ``token_map = (ids, rows, places)`` does the same for some rows only: row ``rows[i]`` of the step takes
        ``ids[places[i]]`` (int32 on the device), the other rows the entries' own ids."""
        ctx = self._build_context(entries, device_tokens, token_map)
        self.last_ctx = ctx          # kept for inspection (which kernels the step's plan chose)
        if self.use_cuda_graphs and not ctx.late_uploads:
            logits = self._forward_graphed(ctx)
        else:
            logits = self._picked(ctx, self.forward(ctx))
        for e in entries:
            self.cache.advance(e.seq_id, len(e.tokens))
        return logits

    def _capture(self, ctx: StepContext):
        """The step's launches recorded into a CUDA graph, on a side stream as capture wants it.  This is what the
        ``torch.cuda.graph`` context does without its preparations (a device synchronisation and the release of every
        cached block of device and pinned memory, about 6 ms, after which the next allocations go to the driver again):
        a server captures dozens of shapes while it runs, and none of them needs the memory that those give back."""
        graph = torch.cuda.CUDAGraph()
        current = ops.torch_stream()
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(self.device)
        side = self._capture_stream
        side.wait_stream(current)
        torch.cuda.set_stream(side)          # (not the `torch.cuda.stream` context: it asks for the current stream without
        try:                                 # naming a device, which makes torch count the devices through the driver)
            if self._graph_pool is None:
                graph.capture_begin()
            else:
                graph.capture_begin(pool=self._graph_pool)
            try:
                out = self.forward(ctx)
            finally:
                graph.capture_end()
        finally:
            torch.cuda.set_stream(current)
        current.wait_stream(side)
        if self._graph_pool is None:
            self._graph_pool = graph.pool()
        return graph, out

    @staticmethod
    def _picked(ctx: StepContext, logits: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """The wanted rows of a row-by-row step's logits (which cover every row of its bucket)."""
        if logits is None or ctx.select_rows is None:
            return logits
        return logits.index_select(0, ctx.select_rows)

    def _forward_graphed(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """A step through a CUDA graph.  The metadata buffer has equal addresses for equal counts, so a
        graph captured for (tokens, requests, wanted rows, block-table width, sizes of the staged index
        arrays and what else the parts named) serves every later step of that shape; only the metadata
        copy stays outside."""
        from ..csrc import ops
        key = (ctx.T, ctx.num_spans, ctx.num_want, ctx.max_pages, ctx.decode_only, tuple(ctx.shape_key))
        hit = self._graphs.get(key)
        if hit is not None:
            self._graphs[key] = self._graphs.pop(key)          # most recently used last
        else:
            seen = self._graph_seen.get(key, 0) + 1
            self._graph_seen[key] = seen
            if len(self._graph_seen) > 4096:              # shapes seen once and never again
                self._graph_seen.clear()
            # A capture costs the host a few milliseconds, as much as several steps.  The shapes of decoding
            # batches and of a lone portion come again hundreds of times; a step that mixes several portions and
            # tokens rarely meets its shape again, so such a shape must have come more often before it is captured.
            settled = ctx.decode_only or ctx.num_spans == 1
            if seen < (2 if settled else self.MIXED_CAPTURE_AFTER):
                return self._picked(ctx, self.forward(ctx))          # the first sights of a shape (also the warm-up)
            if len(self._graphs) >= self.max_graphs:      # the least recently used graph makes room
                del self._graphs[next(iter(self._graphs))]
            before = ops.launch_count()
            graph, out = self._capture(ctx)
            hit = self._graphs[key] = (graph, out, ops.launch_count() - before)
        graph, out, nodes = hit
        graph.replay()
        self.graph_replays += 1
        self.graph_launches += nodes
        if out is None:
            return None
        return out.clone() if ctx.select_rows is None else out.index_select(0, ctx.select_rows)

    def check_device_errors(self) -> None:
        """Raise if a kernel flagged a fault (an id outside the vocabulary reached the device)."""
        from ..csrc import ops
        ops.check_async_errors(self.device)
        if int(self.err.item()) != 0:
            self.err.zero_()
            raise RuntimeError("a kernel reported an out-of-range token id")
