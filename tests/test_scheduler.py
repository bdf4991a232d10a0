"""The scheduler's decisions on the host (no GPU): batch composition against the reference's own
scheduler (golden), one entry per request, page-aware admission, shrinking portions,
preemption when pages run out, and requests that can never fit."""
import json
import os
import random

import pytest

from lightllm_b200.cache import CacheLayout, CacheManager, CacheSpec, KVSpec
from lightllm_b200.engine.scheduler import DECODING, FINISHED, PREFILL, WAITING, Request, Scheduler

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "scheduler_golden.json")


def manager(num_pages, page_size=4, max_seqs=8, max_seq_len=256):
    lo = CacheLayout.build([CacheSpec(kv=KVSpec(1, 8))], [None])
    return CacheManager(lo, page_size, num_pages, max_seqs, max_seq_len)


def run_step(s: Scheduler, next_token=lambda r: 7):
    """Play the engine's part: take the pages, advance, hand back one token per wanting entry."""
    st = s.step()
    s.cache.reserve_all((e.request.id, e.num_tokens) for e in st.entries)
    for e in st.entries:
        s.cache.advance(e.request.id, e.num_tokens)
    sampled = {e.request.id: next_token(e.request) for e in st.entries if e.wants_logits}
    done = s.on_step_done(st, sampled)
    s.cache.check()
    return st, done


def test_batch_composition_equals_the_reference_scheduler():
    g = json.load(open(GOLDEN))
    s = Scheduler(manager(1000), g["chunk_size"], g["max_batch_tokens"], 999)
    for i, (p, n) in enumerate(zip(g["prompts"], g["max_new"])):
        s.add_request(Request(i, [1] * p, max_new_tokens=n, eos_token_id=-1))
    steps = []
    while s.num_active():
        st, _ = run_step(s)
        steps.append([[e.request.id, e.num_tokens, 1 if e.is_prefill else 0] for e in st.entries])
    assert steps == g["steps"]


def test_one_entry_per_request_and_true_positions():
    s = Scheduler(manager(1000), chunk_size=16, max_batch_tokens=32)
    s.add_request(Request(0, [1] * 5, max_new_tokens=3, eos_token_id=-1))
    s.add_request(Request(1, [1] * 40, max_new_tokens=3, eos_token_id=-1))
    st, _ = run_step(s)
    # the reference would emit request 1 twice here (16 + 11); here it appears once
    assert [(e.request.id, e.num_tokens, e.start_pos) for e in st.entries] == [(0, 5, 0), (1, 16, 0)]
    st, _ = run_step(s)
    assert [(e.request.id, e.num_tokens, e.start_pos, e.is_prefill) for e in st.entries] == \
        [(0, 1, 5, False), (1, 16, 16, True)]
    st, _ = run_step(s)
    assert [(e.request.id, e.num_tokens, e.start_pos) for e in st.entries] == [(0, 1, 6), (1, 8, 32)]
    assert st.entries[1].wants_logits
    st, done = run_step(s)
    assert [(e.request.id, e.start_pos, e.is_prefill) for e in st.entries] == [(1, 40, False)]
    assert s.finished[0].finish_reason == "length" and len(s.finished[0].output_tokens) == 3


def test_finish_on_eos_and_pages_come_back():
    m = manager(50)
    s = Scheduler(m, 16, 64)
    s.add_request(Request(0, [1] * 10, max_new_tokens=50, eos_token_id=99))
    toks = iter([5, 6, 99])
    while s.num_active():
        run_step(s, lambda r: next(toks))
    assert s.finished[0].output_tokens == [5, 6, 99] and s.finished[0].finish_reason == "eos"
    assert m.free_pages() == 50 and m.free_slots == 8


def test_admission_waits_for_pages_and_portions_shrink_to_page_edges():
    m = manager(num_pages=6, page_size=4)          # 24 tokens in all
    s = Scheduler(m, chunk_size=16, max_batch_tokens=64)
    s.add_request(Request(0, [1] * 14, max_new_tokens=2, eos_token_id=-1))
    s.add_request(Request(1, [1] * 12, max_new_tokens=2, eos_token_id=-1))
    st, _ = run_step(s)
    # request 0 takes 4 pages; request 1 is admitted with one spare page kept for request 0: 1 page = 4 tokens
    assert [(e.request.id, e.num_tokens) for e in st.entries] == [(0, 14), (1, 4)]
    st, _ = run_step(s)
    assert [(e.request.id, e.num_tokens, e.is_prefill) for e in st.entries][0] == (0, 1, False)
    while s.num_active():
        run_step(s)
    assert all(r.finish_reason == "length" for r in s.finished.values())
    assert m.free_pages() == 6


def test_preemption_when_a_decoding_request_finds_no_page():
    m = manager(num_pages=4, page_size=4)          # 16 tokens
    s = Scheduler(m, chunk_size=16, max_batch_tokens=64)
    s.add_request(Request(0, [1] * 7, max_new_tokens=8, eos_token_id=-1))
    s.add_request(Request(1, [2] * 6, max_new_tokens=8, eos_token_id=-1))
    preempted_at, outputs_before = None, None
    n = 0
    counter = iter(range(100, 1000))
    while s.num_active():
        st, _ = run_step(s, lambda r: next(counter))
        n += 1
        if st.preempted and preempted_at is None:
            preempted_at = n
            assert st.preempted == [1]                       # the request admitted last
            r1 = s.waiting[0]
            assert r1.id == 1 and r1.state == WAITING and r1.num_computed == 0 and r1.preemptions == 1
            outputs_before = list(r1.output_tokens)
            assert outputs_before                             # it had generated something: it is kept
        assert n < 200
    assert preempted_at is not None
    assert s.finished[1].output_tokens[: len(outputs_before)] == outputs_before
    assert len(s.finished[0].output_tokens) == 8 and len(s.finished[1].output_tokens) == 8
    assert m.free_pages() == 4 and m.free_slots == 8


def test_a_request_that_can_never_fit_finishes_with_a_status():
    m = manager(num_pages=4, page_size=4, max_seq_len=64)
    s = Scheduler(m, 16, 64)
    s.add_request(Request(0, [1] * 16, max_new_tokens=4, eos_token_id=-1))       # 16 + 1 > 16 tokens of pool
    assert s.finished[0].finish_reason == "too_long" and s.num_active() == 0
    s.add_request(Request(1, [], max_new_tokens=4))
    assert s.finished[1].finish_reason == "empty_prompt"
    # fits at first, then outgrows the pool while alone: it ends, nothing hangs
    s.add_request(Request(2, [1] * 10, max_new_tokens=50, eos_token_id=-1))
    n = 0
    while s.num_active():
        run_step(s)
        n += 1
        assert n < 100
    assert s.finished[2].finish_reason == "out_of_pages" and len(s.finished[2].output_tokens) == 7
    assert m.free_pages() == 4


def test_max_seq_len_ends_a_request():
    m = manager(num_pages=100, page_size=4, max_seq_len=12)
    s = Scheduler(m, 16, 64)
    s.add_request(Request(0, [1] * 8, max_new_tokens=50, eos_token_id=-1))
    while s.num_active():
        run_step(s)
    assert s.finished[0].finish_reason == "max_seq_len" and s.finished[0].total_len() == 12


def test_budget_and_entry_limits():
    s = Scheduler(manager(1000), chunk_size=8, max_batch_tokens=20, max_prefill_entries=2)
    for i in range(4):
        s.add_request(Request(i, [1] * 30, max_new_tokens=2, eos_token_id=-1))
    st, _ = run_step(s)
    assert [(e.request.id, e.num_tokens) for e in st.entries] == [(0, 8), (1, 8)]       # two prefill entries at most
    s2 = Scheduler(manager(1000), chunk_size=16, max_batch_tokens=20)
    for i in range(3):
        s2.add_request(Request(i, [1] * 30, max_new_tokens=2, eos_token_id=-1))
    st, _ = run_step(s2)
    assert [(e.request.id, e.num_tokens) for e in st.entries] == [(0, 16), (1, 4)] and st.total_tokens() == 20


@pytest.mark.parametrize("seed", range(5))
def test_random_workloads_finish_and_leak_nothing(seed):
    rng = random.Random(seed)
    m = manager(num_pages=rng.randint(12, 40), page_size=4, max_seqs=4, max_seq_len=120)
    s = Scheduler(m, chunk_size=rng.choice([4, 16]), max_batch_tokens=rng.choice([8, 32]))
    reqs = [Request(i, [1] * rng.randint(1, 30), max_new_tokens=rng.randint(1, 20), eos_token_id=-1) for i in range(12)]
    pending = list(reqs)
    n = 0
    while pending or s.num_active():
        if pending and rng.random() < 0.5:
            s.add_request(pending.pop(0))
        if s.num_active():
            st, _ = run_step(s)
            ids = [e.request.id for e in st.entries]
            assert len(ids) == len(set(ids)) and st.total_tokens() <= s.max_batch_tokens + len(ids)
        n += 1
        assert n < 5000
    assert len(s.finished) == 12 and m.free_pages() == m.pools[0].num_pages and m.free_slots == 4
    for r in reqs:
        assert r.state == FINISHED and r.finish_reason in ("length", "too_long", "out_of_pages")
        if r.finish_reason == "length":
            assert len(r.output_tokens) == r.max_new_tokens


def test_a_step_can_be_decided_before_the_last_one_is_read():
    """The accounting in two halves: after ``advance`` (tokens in the cache) the next decode step can be decided,
    ``commit`` adds the sampled tokens later; a request that ends on an end-of-sequence id drops the token of the
    step that was launched ahead; steps that could end a request by length are never launched ahead."""
    m = manager(50)
    s = Scheduler(m, 16, 64)
    s.add_request(Request(0, [1] * 5, max_new_tokens=6, eos_token_id=99))
    s.add_request(Request(1, [2] * 7, max_new_tokens=20, eos_token_id=99))

    def launch():
        st = s.step()
        s.cache.reserve_all((e.request.id, e.num_tokens) for e in st.entries)
        for e in st.entries:
            s.cache.advance(e.request.id, e.num_tokens)
        s.advance(st)
        return st

    first = launch()                                     # both prompts whole, both want logits
    assert s.can_step_ahead(first)                       # a prompt step's successor can be decided too; here it is read first
    assert s.commit(first, {0: 10, 1: 11}) == []
    st1 = launch()                                       # decode step 1
    assert s.can_step_ahead(st1)
    st2 = launch()                                       # decided and launched before st1's tokens are known
    assert [e.start_pos for e in st2.entries] == [e.start_pos + 1 for e in st1.entries]
    assert s.commit(st1, {0: 12, 1: 99}) != []           # request 1 ends on its end-of-sequence id ...
    assert s.finished[1].output_tokens == [11, 99]
    assert not s.can_step_ahead(st2)                   # ... so the batch has changed
    assert s.commit(st2, {0: 13, 1: 55}) == []           # its token of the step launched ahead is dropped
    assert s.finished[1].output_tokens == [11, 99] and s.running[0].output_tokens == [10, 12, 13]
    st3 = launch()
    assert s.can_step_ahead(st3)                       # it samples the 4th of 6 tokens: one more step is safe
    st4 = launch()
    s.commit(st3, {0: 14})
    assert s.can_step_ahead(st4)                       # the 5th; the step after it samples the last
    st5 = launch()
    s.commit(st4, {0: 15})
    assert not s.can_step_ahead(st5)                   # the request ends by length with st5's token
    done = s.commit(st5, {0: 16})
    assert [r.id for r in done] == [0] and s.finished[0].finish_reason == "length"
    assert s.finished[0].output_tokens == [10, 12, 13, 14, 15, 16]
    assert m.free_pages() == 50
    m.check()


def test_steps_with_portions_can_be_decided_ahead_too():
    """``can_step_ahead``: the step after a launched one is decided before its tokens are known whenever no request
    that samples in it can end by length, whatever the step holds: a whole prompt, a portion beside decoded tokens.
    The next step gives the request that has just finished its prompt a decode token at the next position (its id
    comes from the device), goes on with the other prompt's portions, and preempts nobody."""
    m = manager(50)
    s = Scheduler(m, 8, 12)                               # portions of 8 tokens, 12 tokens a step
    s.add_request(Request(0, [1] * 5, max_new_tokens=6, eos_token_id=99))
    s.add_request(Request(1, [2] * 20, max_new_tokens=4, eos_token_id=99))

    def launch():
        st = s.step()
        s.cache.reserve_all((e.request.id, e.num_tokens) for e in st.entries)
        for e in st.entries:
            s.cache.advance(e.request.id, e.num_tokens)
        s.advance(st)
        return st

    st0 = launch()                                        # request 0 whole (5, wants logits) + 7 tokens of request 1
    assert [(e.request.id, e.num_tokens, e.wants_logits) for e in st0.entries] == [(0, 5, True), (1, 7, False)]
    assert s.can_step_ahead(st0)
    st1 = launch()                                        # before st0's token is known
    assert [(e.request.id, e.num_tokens, e.start_pos, e.is_prefill) for e in st1.entries] == [(0, 1, 5, False), (1, 8, 7, True)]
    assert s.running[0].total_len() == 5                  # the token of st0 is not there yet: the entry's id is the device's
    assert s.commit(st0, {0: 10}) == []
    assert s.can_step_ahead(st1) and not st1.preempted
    st2 = launch()
    assert [(e.request.id, e.num_tokens, e.start_pos) for e in st2.entries] == [(0, 1, 6), (1, 5, 15)]
    assert st2.entries[1].wants_logits                    # request 1's prompt ends in this step
    s.commit(st1, {0: 11})
    assert s.can_step_ahead(st2)
    st3 = launch()                                        # both decode; request 1's first token comes from the device
    assert [(e.request.id, e.start_pos, e.is_prefill) for e in st3.entries] == [(0, 7, False), (1, 20, False)]
    s.commit(st2, {0: 12, 1: 30})
    assert s.can_step_ahead(st3)                          # request 0 samples its 4th of 6, request 1 its 2nd of 4
    st4 = launch()
    s.commit(st3, {0: 13, 1: 31})
    assert s.can_step_ahead(st4)                          # request 1 samples its 3rd of 4: the step after samples the last
    st5 = launch()
    s.commit(st4, {0: 14, 1: 32})
    assert not s.can_step_ahead(st5)                      # both end by length with st5's tokens
    done = s.commit(st5, {0: 15, 1: 33})
    assert sorted(r.id for r in done) == [0, 1]
    assert s.finished[0].output_tokens == [10, 11, 12, 13, 14, 15] and s.finished[1].output_tokens == [30, 31, 32, 33]
