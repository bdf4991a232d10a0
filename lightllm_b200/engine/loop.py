"""The serve loop: scheduler -> step function -> sampler, with per-request and per-step metrics.

After the reference's ``BatchMainLoop`` (include/lightllm/engine/batch_loop.h:79-211,
src/engine/batch_loop.cpp:108-305): ``submit`` returns an id at once, ``step`` runs one
scheduler decision through the engine, ``run`` loops until nothing is active; TTFT, TPOT and
latency are kept per request (batch_loop.h:35-60) and the composition of every step
(batch_loop.h:65-74); percentiles interpolate linearly (batch_loop.cpp:369-462).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch

from ..csrc import ops
from ..sampling import Sampler, SamplingParams
from .batch import StepEntry
from .core import EngineCore
from .scheduler import Request, ScheduleStep, Scheduler


@dataclass
class BatchMetrics:
    request_id: int = 0
    prompt_len: int = 0
    output_len: int = 0
    arrival_time_sec: float = 0.0
    first_token_time_sec: float = 0.0
    finish_time_sec: float = 0.0
    finished: bool = False
    first_token_recorded: bool = False
    finish_reason: Optional[str] = None

    def ttft_ms(self) -> float:
        return (self.first_token_time_sec - self.arrival_time_sec) * 1000.0 if self.first_token_recorded else 0.0

    def latency_ms(self) -> float:
        return (self.finish_time_sec - self.arrival_time_sec) * 1000.0

    def tpot_ms(self) -> float:
        if self.output_len <= 0:
            return 0.0
        return (self.finish_time_sec - self.first_token_time_sec) * 1000.0 / self.output_len


@dataclass
class BatchStepMetrics:
    step_number: int = 0
    step_time_sec: float = 0.0
    tokens_processed: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    num_requests: int = 0
    num_prefill_entries: int = 0
    num_decode_entries: int = 0
    active_after: int = 0
    preempted: int = 0


def percentile(values: Sequence[float], p: float) -> float:
    """Linear interpolation between the two nearest ranks (src/engine/batch_loop.cpp:369-386)."""
    if not values:
        return 0.0
    v = sorted(values)
    if len(v) == 1:
        return v[0]
    rank = p / 100.0 * (len(v) - 1)
    lo = int(rank)
    hi = min(lo + 1, len(v) - 1)
    return v[lo] + (v[hi] - v[lo]) * (rank - lo)


class _InFlight:
    """A step that has been launched and whose sampled ids are on their way to the host."""

    __slots__ = ("sched", "wanting", "tokens_dev", "tokens_host", "ready")

    def __init__(self, sched, wanting, tokens_dev, tokens_host, ready):
        self.sched, self.wanting, self.tokens_dev, self.tokens_host, self.ready = sched, wanting, tokens_dev, tokens_host, ready


class BatchMainLoop:
    """One step is kept in flight whenever the next one can be decided without what it samples (no request of it can
    end other than on an end-of-sequence id, every decoding request finds a page; ``Scheduler.can_step_ahead``), whether
    it decodes, carries portions of prompts or both: the next step is launched with the ids that the last one sampled
    still on the device, and the host reads those ids (ends requests on an end-of-sequence id, keeps the metrics)
    while the GPU already runs the next step.  A request that ends this way has computed one token too many, which is
    dropped.  ``decode_ahead=False`` launches and reads back step by step, as the reference does."""

    def __init__(self, engine: EngineCore, chunk_size: int = 16, max_batch_tokens: int = 256,
                 max_prefill_entries: int = 999, decode_ahead: bool = True):
        self.engine = engine
        max_batch_tokens = min(max_batch_tokens, engine.runner.max_batch_tokens)
        self.scheduler = Scheduler(engine.cache, chunk_size, max_batch_tokens, max_prefill_entries)
        self.sampler = Sampler(engine.device)
        self.chunk_size = chunk_size
        self._metrics: Dict[int, BatchMetrics] = {}
        self.step_metrics: List[BatchStepMetrics] = []
        self._requests: Dict[int, Request] = {}
        self._next_id = 0
        self.total_steps = 0
        self._epoch = time.perf_counter()
        self.decode_ahead = decode_ahead
        self._inflight: Optional[_InFlight] = None
        self._pinned = [torch.empty(engine.runner.max_spans, dtype=torch.int32).pin_memory() for _ in range(2)]
        self._pin_turn = 0
        self.steps_ahead = 0             # steps that were launched before their predecessor's ids were read
        self.measure_device = False      # with it, every step is bracketed by events: see device_busy_ms()
        self._device_spans = []

    def wall_clock(self) -> float:
        return time.perf_counter() - self._epoch

    def submit(self, prompt_tokens: Sequence[int], max_new_tokens: int = 64, eos_token_id=None,
               temperature: float = 1.0, top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0,
               seed: int = 42) -> int:
        params = SamplingParams(temperature, top_k, top_p, min_p, seed)
        params.validate()
        if eos_token_id is None:        # the model's own end-of-sequence ids (config.json), none if it names none
            eos_token_id = tuple(getattr(self.engine, "eos_token_ids", ())) or -1
        vocab = self.engine.vocab_size
        for t in prompt_tokens:
            if not 0 <= int(t) < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        rid = self._next_id
        self._next_id += 1
        req = Request(rid, [int(t) for t in prompt_tokens], max_new_tokens=max_new_tokens,
                      eos_token_id=eos_token_id, sampling=params)
        self._requests[rid] = req
        self._metrics[rid] = BatchMetrics(rid, len(req.prompt_tokens), arrival_time_sec=self.wall_clock())
        if max_new_tokens <= 0:
            self.scheduler._finish(req, "length")
        else:
            self.scheduler.add_request(req)
        if req.state == "FINISHED":
            self._record_finish(req)
        return rid

    def has_active(self) -> bool:
        return self.scheduler.num_active() > 0

    def active_count(self) -> int:
        return self.scheduler.num_active()

    def step(self) -> bool:
        """One scheduler decision run through the engine.  False when there was nothing to do."""
        prev = self._inflight
        self._inflight = None
        had_prev = prev is not None
        if prev is not None and not (self.decode_ahead and self.scheduler.can_step_ahead(prev.sched)):
            self._commit(prev)            # the next step depends on what this one sampled: read it first
            prev = None
        sched: ScheduleStep = self.scheduler.step()
        for r in list(self.scheduler.finished.values()):
            if not self._metrics[r.id].finished:
                self._record_finish(r)
        if sched.empty():
            if prev is not None:
                self._commit(prev)
            return had_prev
        if prev is not None and sched.preempted:
            raise RuntimeError("the scheduler preempted a request in a step it had declared predictable")
        # Requests whose last token is still being sampled by the step in flight take it from the device.
        pending = {r.id: i for i, r in enumerate(prev.wanting)} if prev is not None else {}
        entries, wanting, map_rows, map_from = [], [], [], []
        row = 0
        for e in sched.entries:
            r = e.request
            if not e.is_prefill and r.id in pending and e.start_pos >= r.total_len():
                toks = (0,) * e.num_tokens           # placeholders: the ids come from the device
                map_rows.append(row)
                map_from.append(pending[r.id])
            else:
                toks = r.tokens_at(e.start_pos, e.num_tokens)
            entries.append(StepEntry(r.id, toks, [e.num_tokens - 1] if e.wants_logits else []))
            if e.wants_logits:
                wanting.append(r)
            row += e.num_tokens
        token_map = (prev.tokens_dev, map_rows, map_from) if map_rows else None
        flight = self._launch(sched, entries, wanting, token_map=token_map)
        if prev is not None:
            self.steps_ahead += 1
            self._commit(prev)
        if self.decode_ahead and not sched.preempted:
            self._inflight = flight           # read back at the next call, after the next step has been launched
        else:
            self._commit(flight)
        return True

    def _launch(self, sched: ScheduleStep, entries, wanting, token_map=None) -> _InFlight:
        """Run the step and sample; the ids start their way to the host.  The scheduler's first half of the
        accounting (the tokens are in the cache) is done here."""
        if self.measure_device:
            begin = torch.cuda.Event(enable_timing=True)
            begin.record(ops.torch_stream())
        if token_map is None:
            logits = self.engine.step(entries)
        elif token_map[1] == token_map[2] == list(range(len(entries))) and token_map[0].numel() == len(entries) \
                and all(len(e.tokens) == 1 for e in entries):
            logits = self.engine.step(entries, token_map[0])          # a decoding batch: the sampled ids as they are
        else:
            logits = self.engine.step(entries, None, token_map)
        tokens_dev = tokens_host = ready = None
        if wanting:
            tokens_dev = self.sampler.sample_device(logits, [r.id for r in wanting], [r.sampling for r in wanting])
            tokens_host = self._pinned[self._pin_turn][: len(wanting)]
            self._pin_turn ^= 1
            tokens_host.copy_(tokens_dev, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record(ops.torch_stream())
        if self.measure_device:
            end = torch.cuda.Event(enable_timing=True)
            end.record(ops.torch_stream())
            self._device_spans.append((begin, end))
        self.scheduler.advance(sched)
        return _InFlight(sched, wanting, tokens_dev, tokens_host, ready)

    def _commit(self, flight: _InFlight) -> None:
        """The sampled ids are read; requests get their tokens, finish, and the metrics are kept."""
        sched, wanting = flight.sched, flight.wanting
        sampled: Dict[int, int] = {}
        if wanting:
            flight.ready.synchronize()
            sampled = {r.id: t for r, t in zip(wanting, flight.tokens_host.tolist())}
        now = self.wall_clock()
        for r in wanting:
            m = self._metrics[r.id]
            if not m.first_token_recorded:
                m.first_token_recorded, m.first_token_time_sec = True, now
        for r in self.scheduler.commit(sched, sampled):
            self._record_finish(r)
        self.total_steps += 1
        pre = [e for e in sched.entries if e.is_prefill]
        self.step_metrics.append(BatchStepMetrics(
            self.total_steps, now, sched.total_tokens(), sum(e.num_tokens for e in pre),
            len(sched.entries) - len(pre), len(sched.entries), len(pre), len(sched.entries) - len(pre),
            self.scheduler.num_active(), len(sched.preempted)))

    def flush(self) -> None:
        """Read back the step that is still in flight, if any."""
        if self._inflight is not None:
            flight, self._inflight = self._inflight, None
            self._commit(flight)

    def run(self) -> None:
        while self.has_active():
            if not self.step() and self.has_active():
                raise RuntimeError("the scheduler has active requests but schedules nothing")
        self.flush()

    def _record_finish(self, r: Request) -> None:
        m = self._metrics[r.id]
        m.finished, m.finish_time_sec = True, self.wall_clock()
        m.output_len, m.finish_reason = len(r.output_tokens), r.finish_reason
        self.sampler.forget(r.id)

    # ---- results and metrics ---------------------------------------------------------------------
    def generated_tokens(self, request_id: int) -> List[int]:
        self.flush()
        return list(self._requests[request_id].output_tokens)

    def finish_reason(self, request_id: int) -> Optional[str]:
        self.flush()
        return self._requests[request_id].finish_reason

    def metrics(self, request_id: int) -> BatchMetrics:
        return self._metrics[request_id]

    def all_metrics(self) -> List[BatchMetrics]:
        return list(self._metrics.values())

    def total_tokens_generated(self) -> int:
        self.flush()
        return sum(len(r.output_tokens) for r in self._requests.values())

    def _finished(self) -> List[BatchMetrics]:
        return [m for m in self._metrics.values() if m.finished and m.first_token_recorded]

    def stat(self, what: str, p: Optional[float] = None) -> float:
        """``what`` in ttft/tpot/latency; ``p`` a percentile, or None for the mean."""
        vals = [getattr(m, f"{what}_ms")() for m in self._finished()]
        if not vals:
            return 0.0
        return sum(vals) / len(vals) if p is None else percentile(vals, p)

    def device_busy_ms(self) -> float:
        """With ``measure_device``: the time the device spent between the first and the last kernel of every step so
        far, summed; what is missing to the wall clock is the time it waited for the host between steps."""
        torch.cuda.synchronize()
        return sum(b.elapsed_time(e) for b, e in self._device_spans)

    def throughput_tok_s(self) -> float:
        t = self.wall_clock()
        return self.total_tokens_generated() / t if t > 0 else 0.0
