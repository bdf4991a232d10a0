"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees; and decides what happens when pages run out.

Policy: DecodeFirst, as ``DecodeFirstScheduler::step`` (src/engine/scheduler.cpp:34-73): every
decoding request first gets its one token (:38-43), then the budget that is left goes to prompt
portions of at most ``chunk_size`` tokens, oldest request first, at most
``max_prefill_entries`` of them (:46-64).  ``Request`` keeps the reference's fields
(include/lightllm/engine/scheduler.h:23-48).

Differences from the reference, all on purpose:

* a request appears at most once in a step (the reference may cut one prompt into several
  entries of the same step, and its engine then attends wrongly);
* the decode position is the request's true length (the reference's is stale, scheduler.cpp:41);
* the scheduler knows the cache: a request is admitted only when a state slot and the pages of
  its first portion are free beside one spare page for each running request; a portion shrinks
  to the pages that are free;
* when a decoding request needs a page and none is free, the request admitted last is
  preempted: its pages are given back, it returns to the front of the queue, and its prompt
  and the tokens it had generated are computed again later (its output is unchanged);
* a request that can never fit (longer than the pool or than ``max_seq_len``) finishes at once
  with ``finish_reason = "too_long"`` instead of corrupting the cache as the reference does
  (src/engine/engine_server.cpp:1427-1432).
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional

from ..cache import CacheManager
from ..sampling.params import SamplingParams

WAITING, PREFILL, DECODING, FINISHED = "WAITING", "PREFILL", "DECODING", "FINISHED"


@dataclass
class Request:
    id: int
    prompt_tokens: List[int]
    output_tokens: List[int] = field(default_factory=list)
    num_computed: int = 0            # tokens of prompt + output whose keys and values are cached
    max_new_tokens: int = 64
    # The ids that end the sequence: an integer or a collection of them; -1 (no token) means none.  The scheduler
    # knows no vocabulary: callers take the ids from the model's configuration (``eos_token_id`` of config.json).
    eos_token_id: object = -1
    sampling: SamplingParams = field(default_factory=SamplingParams)
    state: str = WAITING
    finish_reason: Optional[str] = None
    preemptions: int = 0

    def all_tokens(self) -> List[int]:
        return self.prompt_tokens + self.output_tokens

    def total_len(self) -> int:
        return len(self.prompt_tokens) + len(self.output_tokens)

    def tokens_at(self, start: int, n: int) -> List[int]:
        """Tokens ``start .. start+n-1`` of prompt + output, without building the whole list."""
        np_ = len(self.prompt_tokens)
        if start >= np_:
            return self.output_tokens[start - np_: start - np_ + n]
        if start + n <= np_:
            return self.prompt_tokens[start: start + n]
        return self.prompt_tokens[start:] + self.output_tokens[: start + n - np_]

    def prefill_remaining(self) -> int:
        return self.total_len() - self.num_computed


@dataclass
class ScheduleEntry:
    request: Request
    num_tokens: int
    start_pos: int
    is_prefill: bool
    wants_logits: bool     # the entry's last token is the request's last: its logits give the next token

    @property
    def request_idx(self) -> int:
        return self.request.id


@dataclass
class ScheduleStep:
    entries: List[ScheduleEntry] = field(default_factory=list)
    preempted: List[int] = field(default_factory=list)

    def total_tokens(self) -> int:
        return sum(e.num_tokens for e in self.entries)

    def empty(self) -> bool:
        return not self.entries


class _Asks:
    """What a step has promised so far: ``(request, tokens)`` pairs and the pages they need in every cache group, kept
    as running totals so that asking whether one more request fits costs one request's arithmetic, not all of them."""

    def __init__(self, cache):
        self.cache = cache
        self.pairs: List[tuple] = []
        self.total = [0] * len(cache.pools)

    def fits(self, seq_id, n: int, spare: int = 0) -> bool:
        """Whether ``n`` more tokens of ``seq_id`` get their pages beside everything promised, with ``spare`` pages
        left free in every group (what ``CacheManager.can_reserve_all`` answers for the whole list)."""
        c = self.cache
        if c.get(seq_id).length + n > c.max_seq_len:
            return False
        need = c.pages_needed(seq_id, n)
        return all(t + x + spare <= p.free_count for t, x, p in zip(self.total, need, c.pools))

    def add(self, seq_id, n: int) -> None:
        for g, x in enumerate(self.cache.pages_needed(seq_id, n)):
            self.total[g] += x
        self.pairs.append((seq_id, n))

    def take_all(self, pairs) -> bool:
        """All of ``pairs`` or none (the list must be empty): the usual case of a decoding batch."""
        c = self.cache
        total = [0] * len(self.total)
        for seq_id, n in pairs:
            if c.get(seq_id).length + n > c.max_seq_len:
                return False
            for g, x in enumerate(c.pages_needed(seq_id, n)):
                total[g] += x
        if not all(t <= p.free_count for t, p in zip(total, c.pools)):
            return False
        self.pairs, self.total = list(pairs), total
        return True

    def drop(self, seq_id) -> None:
        self.pairs = [a for a in self.pairs if a[0] != seq_id]
        self.total = [0] * len(self.total)
        for sid, n in self.pairs:
            for g, x in enumerate(self.cache.pages_needed(sid, n)):
                self.total[g] += x


class Scheduler:
    def __init__(self, cache: CacheManager, chunk_size: int = 16, max_batch_tokens: int = 256,
                 max_prefill_entries: int = 999):
        if chunk_size <= 0 or max_batch_tokens <= 0 or max_prefill_entries <= 0:
            raise ValueError("chunk_size, max_batch_tokens and max_prefill_entries must be positive")
        self.cache = cache
        self.chunk_size = chunk_size
        self.max_batch_tokens = max_batch_tokens
        self.max_prefill_entries = max_prefill_entries
        self.waiting: Deque[Request] = deque()
        self.running: List[Request] = []        # admitted, in admission order (PREFILL or DECODING)
        self.finished: Dict[int, Request] = {}

    # ---- the reference's interface -------------------------------------------------------------
    def add_request(self, req: Request) -> None:
        req.state = WAITING
        limit = min(self.cache.max_seq_len,
                    min(p.num_pages for p in self.cache.pools) * self.cache.page_size if self.cache.pools
                    else self.cache.max_seq_len)
        if not req.prompt_tokens:
            self._finish(req, "empty_prompt")
        elif len(req.prompt_tokens) + 1 > limit:
            self._finish(req, "too_long")
        else:
            self.waiting.append(req)

    def num_active(self) -> int:
        return len(self.waiting) + len(self.running)

    def finish_request(self, req_id: int, reason: str = "stopped") -> None:
        for r in self.running:
            if r.id == req_id:
                self._release(r)
                self._finish(r, reason)
                return
        for r in list(self.waiting):
            if r.id == req_id:
                self.waiting.remove(r)
                self._finish(r, reason)
                return

    # ---- one scheduling decision ---------------------------------------------------------------
    def step(self) -> ScheduleStep:
        out = ScheduleStep()
        cache = self.cache
        budget = self.max_batch_tokens
        asks = _Asks(cache)

        # Priority 1: one token for every decoding request; preempt from the back when pages run out.
        decoding = [r for r in self.running if r.state == DECODING]
        # Fast path: every decoding request gets its token (the usual case).
        if decoding and asks.take_all([(r.id, 1) for r in decoding]):
            out.entries = [ScheduleEntry(r, 1, r.num_computed, False, True) for r in decoding]
            budget -= len(decoding)
            decoding = []
        i = 0
        while i < len(decoding):
            r = decoding[i]
            if asks.fits(r.id, 1):
                asks.add(r.id, 1)
                out.entries.append(ScheduleEntry(r, 1, r.num_computed, False, True))
                budget -= 1
                i += 1
                continue
            victim = self.running[-1]
            if victim is r and len(self.running) == 1:
                # alone and still no page: it has reached what the pool can hold
                self._release(r)
                self._finish(r, "out_of_pages")
                decoding.pop(i)
                continue
            self._preempt(victim, out)
            if victim in decoding:
                j = decoding.index(victim)
                decoding.pop(j)
                if j < i:          # it had already been given its token: take that back
                    asks.drop(victim.id)
                    out.entries = [e for e in out.entries if e.request is not victim]
                    budget += 1
                    i -= 1

        # Priority 2: the budget that is left goes to prompt portions, admitted requests first.
        prefill_count = 0
        for r in [r for r in self.running if r.state == PREFILL]:
            if budget <= 0 or prefill_count >= self.max_prefill_entries:
                break
            n = self._portion(r, budget, asks, spare=0)
            if n > 0:
                self._add_prefill(out, asks, r, n)
                budget -= n
                prefill_count += 1
        while self.waiting and budget > 0 and prefill_count < self.max_prefill_entries:
            r = self.waiting[0]
            if cache.free_slots == 0:
                break
            cache.open(r.id)
            n = self._portion(r, budget, asks, spare=len(self.running))
            if n <= 0:
                cache.close(r.id)
                if not self.running and not out.entries:
                    # nothing else holds pages and it still does not fit: it never will
                    self.waiting.popleft()
                    self._finish(r, "too_long")
                    continue
                break
            self.waiting.popleft()
            r.state = PREFILL
            self.running.append(r)
            self._add_prefill(out, asks, r, n)
            budget -= n
            prefill_count += 1
        return out

    def _portion(self, r: Request, budget: int, asks, spare: int) -> int:
        """Largest portion of ``r`` that the budget, the chunk size and the free pages allow,
        leaving ``spare`` pages free in every group."""
        n = min(self.chunk_size, r.prefill_remaining(), budget)
        cache = self.cache
        while n > 0:
            if asks.fits(r.id, n, spare):
                return n
            # shrink to the next page edge below
            have = cache.get(r.id).length + n
            edge = (have - 1) // cache.page_size * cache.page_size
            n = edge - cache.get(r.id).length
        return 0

    def _add_prefill(self, out: ScheduleStep, asks, r: Request, n: int) -> None:
        asks.add(r.id, n)
        last = r.num_computed + n == r.total_len()
        out.entries.append(ScheduleEntry(r, n, r.num_computed, True, last))

    # ---- after the step ran ----------------------------------------------------------------------
    def on_step_done(self, step: ScheduleStep, sampled: Dict[int, int]) -> List[Request]:
        """Account for a step that ran: ``sampled`` maps a request id to its next token for the
        entries that wanted logits.  Returns the requests that finished."""
        self.advance(step)
        return self.commit(step, sampled)

    def advance(self, step: ScheduleStep) -> None:
        """First half of the accounting, possible as soon as the step has been launched: its tokens are in
        the cache.  A request whose last token was in the step is decoding from now on, although the
        token it sampled is not known yet, so the next step can be decided before ``commit``."""
        for e in step.entries:
            r = e.request
            r.num_computed += e.num_tokens
            if e.wants_logits and r.state != FINISHED:
                r.state = DECODING

    def commit(self, step: ScheduleStep, sampled: Dict[int, int]) -> List[Request]:
        """Second half: the sampled tokens are known.  Requests that finished meanwhile (their token of a
        step that was launched ahead is dropped) are skipped.  Returns the requests that finish now."""
        done = []
        for e in step.entries:
            r = e.request
            if not e.wants_logits or r.state == FINISHED:
                continue
            tok = sampled[r.id]
            r.output_tokens.append(tok)
            reason = None
            eos = r.eos_token_id
            if tok == eos if isinstance(eos, int) else (eos is not None and tok in eos):
                reason = "eos"
            elif len(r.output_tokens) >= r.max_new_tokens:
                reason = "length"
            elif r.total_len() >= self.cache.max_seq_len:
                reason = "max_seq_len"
            if reason:
                self._release(r)
                self._finish(r, reason)
                done.append(r)
        return done

    def can_step_ahead(self, step: ScheduleStep) -> bool:
        """Whether the step after ``step`` (launched, advanced, not yet committed) can be decided now, whatever
        ``step`` held (portions of prompts, decoded tokens, both): none of the requests that are sampling a token in
        it can end with that token other than by an end-of-sequence id, and every decoding request finds room for one
        more token, so that deciding the next step preempts nobody.  (A request that does end on an end-of-sequence id
        has then computed one token too many, which is dropped.)"""
        if step.preempted:
            return False
        limit = self.cache.max_seq_len
        for e in step.entries:
            if not e.wants_logits:
                continue
            r = e.request
            if r.state != DECODING or len(r.output_tokens) + 2 > r.max_new_tokens or r.total_len() + 2 > limit:
                return False
        return self.cache.can_reserve_all([(r.id, 1) for r in self.running if r.state == DECODING])

    # ---- internals ---------------------------------------------------------------------------------
    def _release(self, r: Request) -> None:
        if r in self.running:
            self.running.remove(r)
        if r.id in self.cache.seqs:
            self.cache.close(r.id)

    def _finish(self, r: Request, reason: str) -> None:
        r.state = FINISHED
        r.finish_reason = reason
        self.finished[r.id] = r

    def _preempt(self, r: Request, out: ScheduleStep) -> None:
        self._release(r)
        r.state = WAITING
        r.num_computed = 0
        r.preemptions += 1
        self.waiting.appendleft(r)
        out.preempted.append(r.id)
