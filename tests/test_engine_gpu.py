"""The engine on the GPU beyond replay: generation through the entry point, long decoding, the
first tokens of a sequence, sharp attention over far keys and page edges, preemption, sampling,
each part alone, other arrangements of the run list, and a toy mixer with state of its own that
is registered, built and stepped from here without a change to the framework."""
import math
import os
import random
from dataclasses import dataclass

import numpy as np
import pytest
import torch

from lightllm_b200 import Engine, EngineCore, EngineOptions, StepEntry, write_random_model
from lightllm_b200.cache import CacheLayout, CacheManager, CacheSpec, KVSpec, StateSpec
from lightllm_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry, SubBlock, config_from_dict,
                                  model_spec_for, register_architecture, register_part)
from lightllm_b200.models import Model
from lightllm_b200.parts import (AttentionMixer, CacheView, FeedForward, GatedMLP, LMHead, Mixer, PositionEncoding, RMSNorm,
                                 TokenEmbedding)
from lightllm_b200.weights import WeightSpec, random_tensors, save_file
from tests.plain import qwen2_plain as P
from tests.tiny_configs import PAGE_SIZE, config
from tests.tolerances import atol_for, greedy_margin_for, logits_std, record

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")


def model_dir(tmp_path, name, seed=3, store="float32", edit=None):
    d = str(tmp_path / f"model_{name}_{seed}")
    write_random_model(config(name), seed, d, store)
    if edit:
        cfg, w = P.read_model_dir(d)
        edit(w)
        save_file({k: v.to(torch.float32 if store == "float32" else torch.bfloat16) for k, v in w.items()},
                  os.path.join(d, "model.safetensors"))
    return d


def core_for(d, dtype, page=16, pages=64, max_seqs=4, max_tokens=512):
    return EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=max_tokens, max_batch_tokens=max_tokens,
                                       page_size=page, num_pages=pages, max_seqs=max_seqs))


def sharpen(factor):
    """Scale q and k projections so that attention is sharp: few keys dominate a row, and a key
    that is skipped, stale or at the wrong place changes the logits by far more than rounding.
    The factor is bounded by the plain implementation itself: at 30 its float32 and float64 results
    already differ by 2e-4, at 10 by 3e-6."""
    def edit(w):
        for k in w:
            if k.endswith("q_proj.weight") or k.endswith("k_proj.weight"):
                w[k] = w[k] * factor
    return edit


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype):
    d = model_dir(tmp_path, name, store="float32" if dtype == "float32" else "bfloat16")
    cfg, w = P.read_model_dir(d)
    rng = random.Random(1)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (1, 9, 40, 23)]
    eng = Engine(d, dtype=dtype, max_seq_len=128, max_batch_tokens=32, page_size=PAGE_SIZE[name], num_pages=40,
                 max_seqs=4, chunk_size=16)
    outs, why = eng.generate(prompts, max_new_tokens=10, temperature=0.0, eos_token_id=-1, return_reasons=True)
    assert why == ["length"] * 4 and all(len(o) == 10 for o in outs)
    assert_greedy_follows_plain(cfg, w, prompts, outs, name, dtype)
    eng.core.cache.check()
    assert eng.core.cache.free_pages() == 40


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_steps_replayed_from_graphs_match_steps_launched_one_by_one(tmp_path, dtype):
    """Step shapes that repeat (prompt portions of equal length at equal positions, mixed steps, decode steps) are
    captured in CUDA graphs at their second appearance; with room for two graphs only, graphs are dropped and
    captured again.  The logits are those of a runner that launches every kernel itself."""
    d = model_dir(tmp_path, "A", store="float32" if dtype == "float32" else "bfloat16")
    cfg, _ = P.read_model_dir(d)
    rng = random.Random(11)
    V = cfg["vocab_size"]
    toks = {k: [rng.randrange(V) for _ in range(70)] for k in "abc"}
    outs = {}
    for graphs in (False, True):
        core = core_for(d, dtype, page=PAGE_SIZE["A"], pages=40)
        core.runner.use_cuda_graphs = graphs and core.runner.use_cuda_graphs
        core.runner.max_graphs = 2
        core.runner.MIXED_CAPTURE_AFTER = 2         # mixed shapes too at their second appearance (by default later)
        got = []
        for rnd_ in range(4):                       # the same schedule four times: every shape comes back
            for k in "abc":
                core.open(k)
            got.append(core.step([StepEntry("a", toks["a"][:40], [39])]))
            got.append(core.step([StepEntry("b", toks["b"][:40], [39])]))                       # same shape as the last
            got.append(core.step([StepEntry("a", toks["a"][40:41], [0]), StepEntry("c", toks["c"][:33], [32])]))
            got.append(core.step([StepEntry("a", toks["a"][41:42], [0]), StepEntry("b", toks["b"][40:41], [0]),
                                  StepEntry("c", toks["c"][33:34], [0])]))
            got.append(core.step([StepEntry("a", toks["a"][42:43], [0]), StepEntry("b", toks["b"][41:42], [0]),
                                  StepEntry("c", toks["c"][34:35], [0])]))
            for k in "abc":
                core.close(k)
        outs[graphs] = [g.float().cpu() for g in got]
        if graphs:
            assert core.runner.graph_replays >= 8 and len(core.runner._graphs) <= 2
        core.runner.check_device_errors()
    worst = max(float((a - b).abs().max()) for a, b in zip(outs[False], outs[True]))
    print("largest difference between replayed and launched steps:", worst)
    # the same kernels on the same inputs: equal bits in float32; in bfloat16 the decode contractions add their
    # pieces with float atomics, whose order is free, so the last bits of the float32 sums may differ
    assert worst == 0.0 if dtype == "float32" else worst < 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_ahead_gives_the_same_tokens(tmp_path, dtype):
    """The serve loop that launches a decode step before it has read the last step's ids gives what the
    step-by-step loop gives: with requests of different lengths, requests that arrive while others decode,
    and requests that end on an end-of-sequence id after their next step has already been launched."""
    d = model_dir(tmp_path, "A", store="float32" if dtype == "float32" else "bfloat16")
    cfg, _ = P.read_model_dir(d)
    rng = random.Random(5)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (3, 20, 11, 7)]
    kw = dict(dtype=dtype, max_seq_len=128, max_batch_tokens=32, page_size=PAGE_SIZE["A"], num_pages=40, max_seqs=4,
              chunk_size=16)
    slow = Engine(d, decode_ahead=False, **kw)
    base = slow.generate(prompts, max_new_tokens=24, temperature=0.0, eos_token_id=-1)
    # an id that request 1 produces in mid-stream becomes the end-of-sequence id
    eos = base[1][9]
    results = {}
    for ahead in (False, True):
        eng = Engine(d, decode_ahead=ahead, **kw)
        loop = eng.new_loop()
        ids = [loop.submit(p, max_new_tokens=n, eos_token_id=eos, temperature=0.0)
               for p, n in zip(prompts[:3], (24, 24, 5))]
        for _ in range(6):
            loop.step()
        ids.append(loop.submit(prompts[3], max_new_tokens=9, eos_token_id=eos, temperature=0.0))
        loop.run()
        results[ahead] = ([loop.generated_tokens(i) for i in ids], [loop.finish_reason(i) for i in ids])
        if ahead:
            assert loop.steps_ahead > 5
        eng.core.cache.check()
        assert eng.core.cache.free_pages() == 40
    assert results[True] == results[False]
    assert "eos" in results[True][1] and "length" in results[True][1]
    sampled = {}
    for ahead in (False, True):
        eng = Engine(d, decode_ahead=ahead, **kw)
        sampled[ahead] = eng.generate(prompts, max_new_tokens=12, temperature=0.9, top_k=40, seed=3, eos_token_id=-1)
    assert sampled[True] == sampled[False]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(tmp_path, dtype):
    d = model_dir(tmp_path, "B", store="float32" if dtype == "float32" else "bfloat16")
    cfg, w = P.read_model_dir(d)
    rng = random.Random(2)
    seq = [rng.randrange(1000) for _ in range(230)]
    ref = P.plain_forward(cfg, w, seq)
    core = core_for(d, dtype, page=8, pages=40)
    core.open("x")
    got = [core.step([StepEntry("x", seq[:1], [0])])]                 # the very first token alone
    got.append(core.step([StepEntry("x", seq[1:3], [0, 1])]))          # then two
    for t in range(3, 230):                                            # then 227 single tokens
        got.append(core.step([StepEntry("x", [seq[t]], [0])]))
    got = torch.cat(got).float().cpu()
    err = (got - ref).abs().max(dim=1).values
    tol = atol_for("B", dtype, ref)
    record(f"long decoding tiny B {dtype}", float(err.max()), logits_std(ref))
    assert float(err.max()) <= tol, f"first wrong position {int((err > tol).nonzero()[0])}"
    core.close("x")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_step_with_every_kind_of_span(tmp_path, dtype):
    """One step holds a decoded token over 700 keys, five rows of a prompt over 600 keys, a portion of 100 rows from
    the start and a short new prompt: in bfloat16 they go to the decode kernel, to the tensor-core kernel (the five
    rows too, where all keys are visible; to the CUDA-core kernel in the layer with the window of 150), and to the
    CUDA-core kernel; in float32 the few rows over many keys are walked row by row in pieces.  Sharp attention, so a
    key lost by any of them shows."""
    d = model_dir(tmp_path, "D", seed=12, store="float32" if dtype == "float32" else "bfloat16", edit=sharpen(6.0))
    cfg, w = P.read_model_dir(d)
    V = cfg["vocab_size"]
    rng = random.Random(13)
    seqs = {n: [rng.randrange(V) for _ in range(L)] for n, L in (("a", 702), ("b", 640), ("c", 100), ("d", 7))}
    ref = {n: P.plain_forward(cfg, w, s) for n, s in seqs.items()}
    core = core_for(d, dtype, page=16, pages=120, max_seqs=4, max_tokens=1024)
    for n in seqs:
        core.open(n)
    core.step([StepEntry("a", seqs["a"][:700], [])])
    core.step([StepEntry("b", seqs["b"][:600], [])])
    steps = [
        [("a", 700, 1), ("b", 600, 5), ("c", 0, 100), ("d", 0, 7)],
        [("a", 701, 1), ("b", 605, 35)],
    ]
    worst_seen = [0.0]
    for step in steps:
        lg = core.step([StepEntry(n, seqs[n][at: at + c], list(range(c))) for n, at, c in step]).float().cpu()
        row = 0
        for n, at, c in step:
            err = (lg[row: row + c] - ref[n][at: at + c]).abs().max(dim=1).values
            tol = atol_for("D sharp", dtype, ref)
            worst_seen[0] = max(worst_seen[0], float(err.max()))
            assert float(err.max()) <= tol, \
                f"{dtype}: request {n}: first wrong position {at + int((err > tol).nonzero()[0])}: {float(err.max())}"
            row += c
    record(f"every kind of span, sharp tiny D {dtype}", worst_seen[0], logits_std(ref))
    core.cache.check()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_sharp_attention_over_far_keys_page_edges_and_reused_pages(tmp_path, name, dtype):
    d = model_dir(tmp_path, name, seed=8, store="float32" if dtype == "float32" else "bfloat16",
                  edit=sharpen(10.0 if dtype == "float32" else 6.0))
    cfg, w = P.read_model_dir(d)
    V, page = cfg["vocab_size"], PAGE_SIZE[name]
    rng = random.Random(3)
    maxlen = 120 if name == "A" else 300
    seqs = {i: [rng.randrange(V) for _ in range(n)] for i, n in enumerate([maxlen, 2 * page + 1, 3 * page, 77])}
    ref = {i: P.plain_forward(cfg, w, s) for i, s in seqs.items()}
    core = core_for(d, dtype, page=page, pages=(maxlen + 100) // page + 3, max_seqs=3, max_tokens=maxlen + 8)
    tol = atol_for(name + " sharp", dtype, ref)
    worst_seen = 0.0
    fed = {i: 0 for i in seqs}
    order = [0, 1]
    core.open(0), core.open(1)
    step = 0
    while order:
        entries, exp = [], []
        for i in list(order):
            left = len(seqs[i]) - fed[i]
            n = min(left, rng.choice([1, 2, page - 1, page, page + 1, 2 * page]))
            if left - n == 1:
                n += 1
            entries.append(StepEntry(i, seqs[i][fed[i]: fed[i] + n], list(range(n))))
            exp.append((i, fed[i], n))
            fed[i] += n
        logits = core.step(entries).float().cpu()
        row = 0
        for i, at, n in exp:
            err = (logits[row: row + n] - ref[i][at: at + n]).abs().max()
            worst_seen = max(worst_seen, float(err))
            assert float(err) <= tol, f"{dtype} {name}: step {step}, request {i}, positions {at}..{at + n - 1}: {float(err)}"
            row += n
            if fed[i] == len(seqs[i]):
                core.close(i)
                order.remove(i)
                nxt = [j for j in seqs if fed[j] == 0 and j not in order]
                if nxt:                                   # a new request takes the pages just given back
                    core.open(nxt[0])
                    order.append(nxt[0])
        step += 1
    record(f"sharp attention tiny {name} {dtype}", worst_seen, logits_std(ref))
    core.cache.check()


def test_preemption_keeps_the_output(tmp_path):
    d = model_dir(tmp_path, "A", store="float32")
    rng = random.Random(4)
    prompts = [[rng.randrange(512) for _ in range(n)] for n in (20, 18, 25)]
    roomy = Engine(d, dtype="float32", max_seq_len=128, max_batch_tokens=64, page_size=16, num_pages=40, max_seqs=4)
    want = roomy.generate(prompts, max_new_tokens=30, temperature=0.0, eos_token_id=-1)
    tight = Engine(d, dtype="float32", max_seq_len=128, max_batch_tokens=64, page_size=16, num_pages=7, max_seqs=4)
    got = tight.generate(prompts, max_new_tokens=30, temperature=0.0, eos_token_id=-1)
    assert sum(m.preempted for m in tight.last_loop.step_metrics) > 0
    assert got == want
    assert tight.core.cache.free_pages() == 7


def assert_greedy_follows_plain(cfg, w, prompts, outs, name, dtype):
    """Every generated token is the plain implementation's top-1 for the same history, or the plain top two lie
    within the engine's rounding of each other."""
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o:
            lg = P.plain_forward(cfg, w, seq)[-1]
            top = torch.topk(lg, 2).values
            assert tok == int(torch.argmax(lg)) or float(top[0] - top[1]) < greedy_margin_for(name, dtype, lg), (seq, tok)
            seq.append(tok)


def test_preemption_in_bfloat16_where_the_tensor_core_kernels_run(tmp_path):
    """Pages run out while three requests decode on tiny D (heads of 64: the tensor-core attention and the fused decode
    path): the request admitted last is preempted and computed again later, as a portion this time, and every token
    still follows the plain implementation."""
    d = model_dir(tmp_path, "D", store="bfloat16")
    cfg, w = P.read_model_dir(d)
    rng = random.Random(6)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (40, 35, 50)]
    tight = Engine(d, dtype="bfloat16", max_seq_len=256, max_batch_tokens=128, page_size=16, num_pages=11, max_seqs=4)
    got = tight.generate(prompts, max_new_tokens=40, temperature=0.0, eos_token_id=-1)
    assert sum(m.preempted for m in tight.last_loop.step_metrics) > 0
    assert all(len(o) == 40 for o in got)
    assert_greedy_follows_plain(cfg, w, prompts, got, "D", "bfloat16")
    assert tight.core.cache.free_pages() == 11
    tight.core.runner.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_a_block_table_width_step_with_graphs(tmp_path, dtype):
    """The block table's width in a step is rounded up to 32 pages, so a decoding request keeps its step shape (and
    the graph captured for it) until it enters its 33rd page; there the shape changes and a new graph is captured.
    300 tokens at pages of 8 cross that edge at position 256, with graphs replaying on both sides of it."""
    d = model_dir(tmp_path, "C", store="float32" if dtype == "float32" else "bfloat16")
    cfg, w = P.read_model_dir(d)
    rng = random.Random(14)
    seq = [rng.randrange(cfg["vocab_size"]) for _ in range(300)]
    ref = P.plain_forward(cfg, w, seq)
    core = core_for(d, dtype, page=8, pages=48, max_seqs=2, max_tokens=384)
    assert core.runner.use_cuda_graphs
    core.open("x")
    got = [core.step([StepEntry("x", seq[:236], [235])])]
    widths = set()
    for t in range(236, 300):
        got.append(core.step([StepEntry("x", [seq[t]], [0])]))
        widths.add(-(-(-(-(t + 1) // 8)) // 32) * 32)
    assert widths == {32, 64} and core.runner.graph_replays >= 40
    got = torch.cat(got).float().cpu()
    err = (got - ref[235:]).abs().max(dim=1).values
    tol = atol_for("C", dtype, ref)
    assert float(err.max()) <= tol, f"first wrong position {235 + int((err > tol).nonzero()[0])}: {float(err.max())}"
    core.runner.check_device_errors()


def test_decode_over_many_keys_merged_through_scratch(tmp_path, monkeypatch):
    """From 17 pieces on, the pieces of the decode attention no longer meet inside a cluster but in scratch memory,
    merged by a second kernel.  With the in-cluster limit lowered the engine takes that path at 2,300 keys; sharp
    attention, so a piece that is lost or merged with a wrong weight shows."""
    from lightllm_b200.parts import attention as A
    monkeypatch.setattr(A, "CLUSTER_MERGE_MAX_KEYS", 256)
    raw = config("D")
    raw["max_position_embeddings"] = 4096
    raw["use_sliding_window"] = False
    d = str(tmp_path / "long")
    write_random_model(raw, 15, d, "bfloat16")
    cfg, w = P.read_model_dir(d)
    sharpen(4.0)(w)
    save_file({k: v.to(torch.bfloat16) for k, v in w.items()}, os.path.join(d, "model.safetensors"))
    cfg, w = P.read_model_dir(d)
    rng = random.Random(16)
    seq = [rng.randrange(cfg["vocab_size"]) for _ in range(2312)]
    ref = P.plain_forward(cfg, w, seq)[2300:]
    core = EngineCore(d, EngineOptions(dtype="bfloat16", max_seq_len=4096, max_batch_tokens=1024, page_size=16,
                                       num_pages=160, max_seqs=2))
    core.open("x")
    for at in range(0, 2300, 1000):
        core.step([StepEntry("x", seq[at: min(2300, at + 1000)], [])])
    got = []
    for t in range(2300, 2312):
        got.append(core.step([StepEntry("x", [seq[t]], [0])]))
        plan = next(v for k, v in core.runner.last_ctx.memo.items() if k[0] == "attention_plan")
        assert plan[0] == "decode_mma" and plan[2] > 16, plan[2]
    got = torch.cat(got).float().cpu()
    err = float((got - ref).abs().max())
    record("decode over 2,300 keys merged through scratch, sharp tiny D", err, logits_std(ref))
    assert err <= atol_for("D sharp", "bfloat16", ref), err
    core.runner.check_device_errors()


@pytest.mark.parametrize("name,rows", [("D", 3), ("D", 40), ("E", 17)])
def test_decode_steps_through_the_persistent_kernel(tmp_path, name, rows):
    """Decode steps of several requests with contexts of different lengths (a first token, page edges, the window's
    edge on tiny D) run the layers as one persistent kernel; the logits are the plain implementation's.  With 40
    rows the step is beyond the size up to which the engine chooses that kernel by itself, so the limit is raised."""
    d = model_dir(tmp_path, name, seed=17, store="bfloat16", edit=sharpen(4.0))
    cfg, w = P.read_model_dir(d)
    rng = random.Random(18)
    V, page = cfg["vocab_size"], PAGE_SIZE[name]
    lens = [1 + (37 * i) % 200 for i in range(rows)]
    lens[0], lens[-1] = 1, 2 * page          # a request whose first token is decoded alone; one at a page's edge
    seqs = {i: [rng.randrange(V) for _ in range(n + 6)] for i, n in enumerate(lens)}
    ref = {i: P.plain_forward(cfg, w, s) for i, s in seqs.items()}
    core = EngineCore(d, EngineOptions(dtype="bfloat16", max_seq_len=256, max_batch_tokens=512, page_size=page,
                                       num_pages=rows * (-(-206 // page) + 1), max_seqs=rows))
    assert core.runner.fused.enabled and core.runner.fused.segment_at(0).end == cfg["num_hidden_layers"]
    core.runner.fused.max_rows = 64
    for i, n in enumerate(lens):
        core.open(i)
        if n > 1:
            core.step([StepEntry(i, seqs[i][: n - 1], [])])
    before = core.launch_count()
    tol = atol_for(name + " sharp", "bfloat16", ref)
    worst = 0.0
    for t in range(6):
        lg = core.step([StepEntry(i, [seqs[i][lens[i] - 1 + t]], [0]) for i in range(rows)]).float().cpu()
        for i in range(rows):
            err = float((lg[i] - ref[i][lens[i] - 1 + t]).abs().max())
            worst = max(worst, err)
            assert err <= tol, f"tiny {name}: step {t}, request {i} at position {lens[i] - 1 + t}: {err}"
    record(f"persistent decode tiny {name} {rows} rows", worst, logits_std(ref))
    # embedding, rotation table, the layers, final norm, head: five launches a step (the first steps are not yet graphs)
    assert core.launch_count() - before <= 8 * 6
    core.runner.check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["C", "D", "E"])
def test_small_mixed_steps_described_row_by_row(tmp_path, monkeypatch, name, dtype):
    """Steps of few rows that mix portions and decoded tokens are given to the kernels row by row (every token a span
    of its own): the logits follow the plain implementation as they do with the portions kept whole, the step has the
    shape of a decoding batch, and two steps of different composition but as many rows and wanted places replay one
    CUDA graph.  C has a window on its upper layers (two cache groups), D heads of 64 with a window, E heads of 128."""
    d = model_dir(tmp_path, name, seed=31, store="float32" if dtype == "float32" else "bfloat16", edit=sharpen(3.0))
    cfg, w = P.read_model_dir(d)
    rng = random.Random(32)
    V, page = cfg["vocab_size"], PAGE_SIZE[name]
    seqs = {i: [rng.randrange(V) for _ in range(120)] for i in range(5)}
    ref = {i: P.plain_forward(cfg, w, s) for i, s in seqs.items()}
    tol = atol_for({"C": "C sharp"}.get(name, name + " sharp"), dtype, ref)

    def run(rowwise: bool):
        monkeypatch.setenv("LLB_ROWWISE_STEPS", "1" if rowwise else "0")
        core = EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=256, max_batch_tokens=256, page_size=page,
                                           num_pages=6 * (-(-128 // page) + 1), max_seqs=6))
        for i in range(5):
            core.open(i)
        got, shapes = [], []
        at = {i: 0 for i in range(5)}

        def step(parts):             # parts: (request, tokens, wanted places)
            entries = []
            for i, n, want in parts:
                entries.append(StepEntry(i, seqs[i][at[i]: at[i] + n], want))
            out = core.step(entries)
            ctx = core.runner.last_ctx
            shapes.append((ctx.T, ctx.num_spans, ctx.decode_only))
            k = 0
            for i, n, want in parts:
                for wpl in want:
                    got.append((i, at[i] + wpl, out[k].float().cpu()))
                    k += 1
                at[i] += n
        step([(0, 70, [69]), (1, 40, [39])])                 # long enough to stay portions: 110 rows
        step([(0, 1, [0]), (1, 1, [0]), (2, 17, [16])])      # 19 rows, three wanted
        step([(0, 1, [0]), (2, 1, [0]), (3, 17, [16])])      # other requests, the same counts: the same shape
        step([(0, 1, [0]), (2, 1, [0]), (4, 17, [16])])      # third sight: replayed
        step([(3, 2, [0, 1]), (4, 5, [4]), (1, 3, [2])])     # portions only, down to two tokens
        step([(i, 1, [0]) for i in range(5)])                # a plain decoding batch
        core.runner.check_device_errors()
        return got, shapes, core.runner.graph_replays

    row, shapes_row, replays_row = run(True)
    whole, shapes_whole, _ = run(False)
    # (row by row a step is padded to a multiple of eight rows by repeating its last row)
    assert shapes_row == [(110, 2, False), (24, 24, True), (24, 24, True), (24, 24, True), (16, 16, True), (5, 5, True)]
    assert shapes_whole == [(110, 2, False), (19, 3, False), (19, 3, False), (19, 3, False), (10, 3, False), (5, 5, True)]
    assert replays_row >= 2          # the shape of 19 rows is captured at its second sight and replayed at its third
    worst = 0.0
    for (i, pos, a), (j, pos2, b) in zip(row, whole):
        assert (i, pos) == (j, pos2)
        worst = max(worst, float((a - ref[i][pos]).abs().max()), float((b - ref[i][pos]).abs().max()))
    assert worst <= tol, worst


def test_token_ids_taken_from_the_device(tmp_path):
    """``step(entries, device_tokens)`` reads the step's ids from a device tensor (the entries only give the counts):
    a decoding batch, and a small mixed step that is described row by row and padded, where the padding has to
    repeat the last row's id.  The logits equal those of the same steps with the ids in the entries."""
    d = model_dir(tmp_path, "E", seed=5, store="bfloat16")
    cfg, w = P.read_model_dir(d)
    rng = random.Random(6)
    V = cfg["vocab_size"]
    seqs = {i: [rng.randrange(V) for _ in range(60)] for i in range(3)}

    def run(on_device: bool):
        core = EngineCore(d, EngineOptions(dtype="bfloat16", max_seq_len=128, max_batch_tokens=128, page_size=16,
                                           num_pages=32, max_seqs=4, use_cuda_graphs=False))
        for i in range(3):
            core.open(i)

        def step(parts):
            ids = [t for i, a, b, _ in parts for t in seqs[i][a:b]]
            if on_device:
                dev = torch.tensor(ids, dtype=torch.int32, device="cuda")
                entries = [StepEntry(i, [0] * (b - a), want) for i, a, b, want in parts]       # placeholders of the right count
                return core.step(entries, dev).float().cpu()
            return core.step([StepEntry(i, seqs[i][a:b], want) for i, a, b, want in parts]).float().cpu()
        out = [step([(0, 0, 30, [29]), (1, 0, 20, [19])])]
        out.append(step([(0, 30, 31, [0]), (1, 20, 21, [0]), (2, 0, 11, [10])]))          # 13 rows: row by row, padded to 16
        assert core.runner.last_ctx.rowwise and core.runner.last_ctx.T == 16
        out.append(step([(0, 31, 32, [0]), (1, 21, 22, [0]), (2, 11, 12, [0])]))          # a decoding batch
        core.runner.check_device_errors()
        return out

    # the same kernels over the same numbers: what may differ is the order in which split contractions add their pieces
    # (a quarter of the allowance against the plain implementation, as where the step executor is compared with the parts)
    ref = {i: P.plain_forward(cfg, w, s) for i, s in seqs.items()}
    tol = atol_for("E", "bfloat16", ref)
    for a, b in zip(run(False), run(True)):
        assert a.shape == b.shape and float((a - b).abs().max()) <= 0.25 * tol


@pytest.mark.parametrize("rowwise", ["1", "0"])
def test_some_rows_take_their_ids_from_the_device(tmp_path, monkeypatch, rowwise):
    """``step(entries, None, (ids, rows, places))``: some rows of a mixed step (the decoded tokens of requests whose
    last id a step in flight is still sampling) take their ids from a device tensor, the rest from the entries.  The
    same shape of step comes nine times, with none, one or both of its decoded rows mapped, so that its CUDA graph is
    captured on the way and replayed with maps of other lengths: no array that the graph reads may move with the map.
    With the portions kept whole the step's attention items are staged behind the fixed arrays, which is where a map
    of varying length once pushed them aside."""
    monkeypatch.setenv("LLB_ROWWISE_STEPS", rowwise)
    d = model_dir(tmp_path, "E", seed=9, store="bfloat16")
    cfg, w = P.read_model_dir(d)
    rng = random.Random(10)
    V = cfg["vocab_size"]
    seqs = {i: [rng.randrange(V) for _ in range(120)] for i in range(3)}
    ref = {i: P.plain_forward(cfg, w, s) for i, s in seqs.items()}
    tol = atol_for("E", "bfloat16", ref)
    core = EngineCore(d, EngineOptions(dtype="bfloat16", max_seq_len=256, max_batch_tokens=128, page_size=16,
                                       num_pages=40, max_seqs=4))
    at = {0: 40, 1: 35, 2: 0}
    for i in range(3):
        core.open(i)
    core.step([StepEntry(0, seqs[0][:40], []), StepEntry(1, seqs[1][:35], [])])
    worst = 0.0
    for n in range(9):
        mapped = [(0, 1), (0,), (), (1,)][n % 4]            # which of the two decoded rows take their id from the device
        ids_dev = torch.tensor([seqs[1][at[1]], 7, seqs[0][at[0]]], dtype=torch.int32, device="cuda")   # places 0 and 2 are used
        place = {0: 2, 1: 0}
        entries = [StepEntry(i, [0] if i in mapped else [seqs[i][at[i]]], [0]) for i in (0, 1)]
        entries.append(StepEntry(2, seqs[2][at[2]: at[2] + 8], []))
        token_map = (ids_dev, [i for i in (0, 1) if i in mapped], [place[i] for i in (0, 1) if i in mapped]) if mapped else None
        out = core.step(entries, None, token_map).float().cpu()
        for k, i in enumerate((0, 1)):
            worst = max(worst, float((out[k] - ref[i][at[i]]).abs().max()))
            at[i] += 1
        at[2] += 8
    core.runner.check_device_errors()
    assert core.runner.graph_replays >= 3
    assert worst <= tol, worst


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "D", "E"])
def test_layers_through_the_step_executor_match_the_parts(tmp_path, monkeypatch, name, dtype):
    """The same steps (a whole prompt, portions beside decoded tokens, decode steps of few and of 40 rows, a step whose
    portion is long enough for the tensor-core projection) through the library's step executor and through the parts
    launched one by one: the two issue the same kernels, so the logits agree to the last bits that the order of
    atomic adds leaves open, and both follow the plain implementation."""
    d = model_dir(tmp_path, name, seed=23, store="float32" if dtype == "float32" else "bfloat16", edit=sharpen(3.0))
    cfg, w = P.read_model_dir(d)
    rng = random.Random(24)
    V, page = cfg["vocab_size"], PAGE_SIZE[name]
    nreq = 40
    lens = [3 + (29 * i) % 90 for i in range(nreq)]
    seqs = {i: [rng.randrange(V) for _ in range(n + 4)] for i, n in enumerate(lens)}
    seqs["long"] = [rng.randrange(V) for _ in range(150)]
    ref = {i: P.plain_forward(cfg, w, s) for i, s in seqs.items()}

    def run(native: bool):
        monkeypatch.setenv("LLB_NATIVE_STEP", "1" if native else "0")
        monkeypatch.setenv("LLB_FUSED_DECODE", "0")          # decode steps take the layer-by-layer path as well
        monkeypatch.setenv("LLB_ROWWISE_STEPS", "0")         # and small mixed steps keep their portions (the parts' plan)
        core = EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=256, max_batch_tokens=2048, page_size=page,
                                           num_pages=(nreq + 2) * (-(-160 // page) + 1), max_seqs=nreq + 1,
                                           use_cuda_graphs=False))
        assert all(core.runner.native.covers) == native
        out = []
        for i in range(nreq):
            core.open(i)
        core.open("long")
        # whole prompts of the first requests, one by one and several in a step
        out.append(core.step([StepEntry(0, seqs[0][: lens[0]], [lens[0] - 1])]))
        out.append(core.step([StepEntry(i, seqs[i][: lens[i]], [lens[i] - 1]) for i in range(1, 6)]))
        # portions of the long prompt beside decoded tokens of those, then beside more prompts
        out.append(core.step([StepEntry("long", seqs["long"][:100], [0, 99])] +
                             [StepEntry(i, [seqs[i][lens[i]]], [0]) for i in range(0, 6)]))
        out.append(core.step([StepEntry("long", seqs["long"][100:150], [49])] +
                             [StepEntry(i, seqs[i][: lens[i]], [lens[i] - 1]) for i in range(6, nreq)]))
        # decode steps: three rows, then forty
        out.append(core.step([StepEntry(i, [seqs[i][lens[i] + 1]], [0]) for i in range(0, 3)]))
        out.append(core.step([StepEntry(i, [seqs[i][lens[i] + (2 if i < 3 else 1 if i < 6 else 0)]], [0]) for i in range(nreq)]))
        core.runner.check_device_errors()
        calls = core.runner.native.calls
        return [o.float().cpu() for o in out], calls

    parts, calls0 = run(False)
    native, calls1 = run(True)
    assert calls0 == 0 and calls1 == 6          # one call of the executor per step
    tol = atol_for({"B": "C sharp"}.get(name, name + " sharp"), dtype, ref)
    # In bfloat16 the split contractions add their pieces in whatever order they arrive; a float sum that differs in its
    # last bit can round an activation to the neighbouring bfloat16, so the two runs may differ by a fraction of the
    # error that either has against the plain implementation (a quarter of the allowance, half of the measured worst).
    for a, b in zip(parts, native):
        assert a.shape == b.shape
        assert float((a - b).abs().max()) <= (1e-5 if dtype == "float32" else 0.25 * tol)
    # and against the plain implementation: the first and the last step
    assert float((native[0][0] - ref[0][lens[0] - 1]).abs().max()) <= tol
    last = native[-1]
    for i in range(nreq):
        at = lens[i] + (2 if i < 3 else 1 if i < 6 else 0)
        assert float((last[i] - ref[i][at]).abs().max()) <= tol, (i, at)


def test_temperature_sampling_is_seeded_and_per_request(tmp_path):
    d = model_dir(tmp_path, "A", store="bfloat16")
    eng = Engine(d, dtype="bfloat16", max_seq_len=128, max_batch_tokens=64, num_pages=40, max_seqs=4)
    p = [[5, 6, 7, 8], [9, 10, 11]]
    a = eng.generate(p, max_new_tokens=12, temperature=1.0, top_k=50, top_p=0.95, seed=7, eos_token_id=-1)
    b = eng.generate(p, max_new_tokens=12, temperature=1.0, top_k=50, top_p=0.95, seed=7, eos_token_id=-1)
    c = eng.generate(p, max_new_tokens=12, temperature=1.0, top_k=50, top_p=0.95, seed=8, eos_token_id=-1)
    alone = eng.generate(p[:1], max_new_tokens=12, temperature=1.0, top_k=50, top_p=0.95, seed=7, eos_token_id=-1)
    assert a == b and a != c
    assert alone[0] == a[0]                       # what else is in the batch does not change a request's draws
    greedy = eng.generate(p, max_new_tokens=12, temperature=0.0, eos_token_id=-1)
    assert greedy != a


def test_step_errors_leave_the_cache_as_it_was(tmp_path):
    from lightllm_b200.cache import OutOfPages
    from lightllm_b200.engine import StepError
    d = model_dir(tmp_path, "A")
    core = core_for(d, "float32", pages=2, max_tokens=64)
    core.open("a"), core.open("b")
    with pytest.raises(StepError, match="outside the vocabulary"):
        core.step([StepEntry("a", [1, 512], [])])
    with pytest.raises(StepError, match="twice"):
        core.step([StepEntry("a", [1], []), StepEntry("a", [2], [])])
    with pytest.raises(OutOfPages):
        core.step([StepEntry("a", [1] * 20, []), StepEntry("b", [1] * 20, [])])
    assert core.cache.free_pages() == 2 and core.cache.get("a").length == 0
    assert core.step([StepEntry("a", [1] * 20, [19])]).shape == (1, 512)


# ---------------------------------------------------------------------------------------------
# Each part alone
# ---------------------------------------------------------------------------------------------
def bound(part, dtype, seed=0, scale=None):
    t = random_tensors(part.weight_specs(), seed, torch.float32)
    if scale:
        t = {k: v * scale for k, v in t.items()}
    dev = {k: v.to(dtype if v.ndim > 1 else torch.float32).to(DEV) for k, v in t.items()}
    part.bind(dev, dtype, DEV)
    return {k: v.to(dtype).float() if v.ndim > 1 else v for k, v in t.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_parts_alone(dtype):
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    g = torch.Generator().manual_seed(5)
    D, I, V, T = 72, 100, 333, 13
    emb = TokenEmbedding("e", V, D)
    w = bound(emb, dtype)
    ids = torch.randint(0, V, (T,), generator=g, dtype=torch.int32)
    h = emb.forward(ids.to(DEV))
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), P.plain_embedding(ids, w["e.weight"]))
    norm = RMSNorm("n", D, 3e-5)
    wn = bound(norm, dtype)
    x = norm.forward(h * 50)
    assert x.dtype == dtype
    ref_x = P.plain_rmsnorm(h.cpu() * 50, wn["n.weight"], 3e-5)
    assert torch.allclose(x.float().cpu(), ref_x, atol=tol, rtol=tol)
    rows = torch.tensor([4, 0], dtype=torch.int32, device=DEV)
    assert torch.allclose(norm.forward_rows(h * 50, rows).float().cpu(), ref_x[[4, 0]], atol=tol, rtol=tol)
    ffn = GatedMLP("f", D, I)
    wf = bound(ffn, dtype, scale=5.0)
    res = torch.zeros((T, D), dtype=torch.float32, device=DEV)
    ffn.forward(x, res)
    ref = P.plain_swiglu(x.float().cpu(), wf["f.gate_proj.weight"], wf["f.up_proj.weight"], wf["f.down_proj.weight"])
    assert torch.allclose(res.cpu(), ref, atol=tol * float(ref.abs().max()), rtol=tol)
    head = LMHead("h", V, D)
    wh = bound(head, dtype)
    lg = head.forward(x)
    assert lg.dtype == torch.float32
    assert torch.allclose(lg.cpu(), P.plain_linear(x.float().cpu(), wh["h.weight"]), atol=tol, rtol=tol)


class HandContext:
    """A step context made by hand for one mixer: spans over a cache manager."""

    def __init__(self, cache, spans, dtype):
        from lightllm_b200.engine.batch import Span, StepContext
        ctx = StepContext()
        rows, sp = 0, []
        for sid, n in spans:
            seq = cache.get(sid)
            cache.reserve(sid, n)
            sp.append(Span(sid, seq.slot, seq.length, n, rows))
            rows += n
        i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
        ctx.T, ctx.spans = rows, sp
        ctx.positions = i32([s.start + j for s in sp for j in range(s.length)])
        ctx.span_row, ctx.span_len = i32([s.row for s in sp]), i32([s.length for s in sp])
        ctx.span_pos, ctx.span_slot = i32([s.start for s in sp]), i32([s.slot for s in sp])
        ctx.iota, ctx.zeros = i32(list(range(len(sp)))), i32([0] * len(sp))
        P_ = cache.max_pages_per_seq
        bt = torch.full((len(sp), P_), -1, dtype=torch.int32)
        for i, s in enumerate(sp):
            t = cache.block_table(s.seq_id, 0)
            bt[i, : len(t)] = torch.tensor(t, dtype=torch.int32)
        ctx.block_tables = [bt.to(DEV)]
        ctx.slot_mapping = [i32([x for s in sp for x in cache.slot_mapping(s.seq_id, 0, s.start, s.length)])]
        ctx.max_pages, ctx.page_size = P_, cache.page_size
        ctx.decode_only = all(s.length == 1 for s in sp)
        ctx.max_context = max(s.start + s.length for s in sp)
        ctx.dtype, ctx.device, ctx.cache = dtype, DEV, cache
        self.ctx, self.cache, self.spans = ctx, cache, spans

    def done(self):
        for sid, n in self.spans:
            self.cache.advance(sid, n)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("style,rotary_dim,window", [("neox", 24, None), ("interleaved", 16, 9)])
def test_attention_mixer_alone(dtype, style, rotary_dim, window):
    """The mixer with its own sizes (5 heads in groups of 5, head 24, partial rotary), fed in
    portions beside a decoding request, against the plain parts on whole sequences."""
    D, Hq, Hkv, hd, page = 40, 5, 1, 24, 4
    mixer = AttentionMixer("a", D, Hq, Hkv, hd, position=PartSpec("rotary", {
        "head_dim": hd, "theta": 777.0, "rotary_dim": rotary_dim, "style": style}), window=window, out_bias=True)
    w = bound(mixer, dtype, scale=4.0)
    layout = CacheLayout.build([mixer.cache_spec()], [None])
    cache = CacheManager(layout, page, 30, 3, 80, dtype, DEV)
    k, v = cache.plane_kv(0, 0)
    view = CacheView(0, k, v, None, True)
    g = torch.Generator().manual_seed(6)
    xs = {"p": torch.randn(37, D, generator=g).to(dtype), "q": torch.randn(21, D, generator=g).to(dtype)}

    def plain(x):
        T = x.shape[0]
        x = x.float()
        pos = torch.arange(T)
        lin = lambda n, b=True: P.plain_linear(x, w[f"a.{n}_proj.weight"], w.get(f"a.{n}_proj.bias") if b else None)
        q = P.plain_rope(lin("q").reshape(T, Hq, hd), pos, 777.0, rotary_dim, style == "interleaved")
        kk = P.plain_rope(lin("k").reshape(T, Hkv, hd), pos, 777.0, rotary_dim, style == "interleaved")
        a = P.plain_attention(q, kk, lin("v").reshape(T, Hkv, hd), 1 / math.sqrt(hd), window)
        return P.plain_linear(a.reshape(T, Hq * hd), w["a.o_proj.weight"], w["a.o_proj.bias"])

    ref = {n: plain(x) for n, x in xs.items()}
    cache.open("p"), cache.open("q")
    fed = {"p": 0, "q": 0}
    plan = [[("p", 9), ("q", 20)], [("p", 2), ("q", 1)], [("p", 13)], [("p", 1)], [("p", 12)]]
    tol = 2e-5 if dtype == torch.float32 else 4e-2
    for feeds in plan:
        hc = HandContext(cache, feeds, dtype)
        x = torch.cat([xs[n][fed[n]: fed[n] + c] for n, c in feeds]).to(DEV)
        res = torch.zeros((x.shape[0], D), dtype=torch.float32, device=DEV)
        mixer.forward(x, res, hc.ctx, view)
        hc.done()
        want = torch.cat([ref[n][fed[n]: fed[n] + c] for n, c in feeds])
        assert torch.allclose(res.cpu(), want, atol=tol * float(want.abs().max()), rtol=tol), feeds
        for n, c in feeds:
            fed[n] += c


# ---------------------------------------------------------------------------------------------
# Other arrangements of the same parts, and a toy mixer with state of its own
# ---------------------------------------------------------------------------------------------
class ToyStateMixer(Mixer):
    """A mixer with a fixed-size state per request and no pages: s_t = decay * s_{t-1} + x_t and
    out_t = s_t W^T.  Defined here, not in the framework."""

    def __init__(self, prefix, hidden_size, decay):
        self.prefix, self.hidden_size, self.decay = prefix, hidden_size, float(decay)
        self.w = None

    def cache_spec(self):
        return CacheSpec(state=StateSpec((self.hidden_size,), "float32"))

    def weight_specs(self):
        return [WeightSpec(f"{self.prefix}.mix.weight", (self.hidden_size, self.hidden_size), init=("normal", 0.05))]

    def bind(self, tensors, dtype, device):
        self.w = tensors[f"{self.prefix}.mix.weight"].float()

    def forward(self, x, residual, ctx, cache):
        for s in ctx.spans:
            state = cache.state[s.slot]
            if s.start == 0:
                state.zero_()
            for t in range(s.row, s.row + s.length):
                state.mul_(self.decay).add_(x[t].float())
                residual[t] += state @ self.w.t()


class ToyRoutedFFN(FeedForward):
    """A feed-forward with routing: router logits in float, the ``top_k`` largest experts, their softmax as
    weights; an expert is ``down(relu(up(x)))``.  Defined here, not in the framework."""

    def __init__(self, prefix, hidden_size, inner, experts, top_k):
        self.prefix, self.D, self.inner, self.E, self.top_k = prefix, hidden_size, inner, experts, top_k

    def weight_specs(self):
        specs = [WeightSpec(f"{self.prefix}.router.weight", (self.E, self.D), init=("normal", 0.5))]
        for e in range(self.E):
            specs.append(WeightSpec(f"{self.prefix}.experts.{e}.up.weight", (self.inner, self.D), init=("normal", 0.1)))
            specs.append(WeightSpec(f"{self.prefix}.experts.{e}.down.weight", (self.D, self.inner), init=("normal", 0.1)))
        return specs

    def bind(self, tensors, dtype, device):
        self.router = tensors[f"{self.prefix}.router.weight"].float()
        self.up = [tensors[f"{self.prefix}.experts.{e}.up.weight"] for e in range(self.E)]
        self.down = [tensors[f"{self.prefix}.experts.{e}.down.weight"] for e in range(self.E)]

    def forward(self, x, residual, ctx):
        logits = x.float() @ self.router.t()
        top_v, top_i = logits.topk(self.top_k, dim=-1)
        weight = torch.softmax(top_v, dim=-1)
        for e in range(self.E):
            rows, slot = (top_i == e).nonzero(as_tuple=True)
            if rows.numel():
                y = torch.relu(x[rows] @ self.up[e].t()) @ self.down[e].t()
                residual.index_add_(0, rows, y.float() * weight[rows, slot].unsqueeze(1))


class ToyLearnedPosition(PositionEncoding):
    """Another position encoding: a learned vector per position added to every head's q and another to its k."""

    def __init__(self, prefix, head_dim, max_positions):
        self.prefix, self.head_dim, self.max_positions = prefix, head_dim, max_positions

    def weight_specs(self):
        return [WeightSpec(f"{self.prefix}.q_pos", (self.max_positions, self.head_dim), init=("normal", 0.5)),
                WeightSpec(f"{self.prefix}.k_pos", (self.max_positions, self.head_dim), init=("normal", 0.5))]

    def bind(self, tensors, dtype, device):
        self.q_pos, self.k_pos = tensors[f"{self.prefix}.q_pos"].float(), tensors[f"{self.prefix}.k_pos"].float()

    def apply(self, q, k, positions):
        at = positions.long()
        q = q + self.q_pos[at].unsqueeze(1)
        return q, (None if k is None else k + self.k_pos[at].unsqueeze(1))


@dataclass(frozen=True)
class ToyConfig(ModelConfig):
    hidden_size: int = 0
    vocab_size: int = 0
    heads: int = 0
    kv_heads: int = 0
    head_dim: int = 0
    inner: int = 0
    decay: float = 0.5
    eps: float = 1e-6
    variant: str = "state"

    @staticmethod
    def from_dict(raw, where="config.json"):
        return ToyConfig(architecture=raw["architectures"][0], raw=dict(raw), hidden_size=raw["width"],
                         vocab_size=raw["vocab"], heads=raw["heads"], kv_heads=raw["kv_heads"],
                         head_dim=raw["head_dim"], inner=raw["inner"], decay=raw.get("decay", 0.5),
                         eps=raw.get("eps", 1e-6), variant=raw.get("variant", "state"))


ROUTED = {"experts": 5, "top_k": 2, "inner": 40, "max_positions": 128}


def toy_spec(cfg: ToyConfig) -> ModelSpec:
    D = cfg.hidden_size
    norm = lambda p: PartSpec("rmsnorm", {"hidden_size": D, "eps": cfg.eps}, p)
    attn = lambda p: PartSpec("attention", {"hidden_size": D, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads,
                                            "head_dim": cfg.head_dim, "qkv_bias": False,
                                            "position": PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": 100.0})}, p)
    ffn = lambda p: PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": cfg.inner}, p)
    if cfg.variant == "state":
        layers = [LayerSpec(norm("l0.n1"), PartSpec("toy_state", {"hidden_size": D, "decay": cfg.decay}, "l0.toy"),
                            norm("l0.n2"), ffn("l0.ffn")),
                  LayerSpec(norm("l1.n1"), attn("l1.attn"), norm("l1.n2"), ffn("l1.ffn"))]
        run = [RunEntry(0), RunEntry(1)]
    elif cfg.variant == "routed":   # learned positions in the first layer's attention, routed experts in the last layer
        learned = PartSpec("attention", {"hidden_size": D, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads,
                                         "head_dim": cfg.head_dim, "qkv_bias": False,
                                         "position": PartSpec("toy_learned", {"head_dim": cfg.head_dim,
                                                                              "max_positions": ROUTED["max_positions"]},
                                                              "l0.attn.pos")}, "l0.attn")
        moe = PartSpec("toy_routed", {"hidden_size": D, "inner": ROUTED["inner"], "experts": ROUTED["experts"],
                                      "top_k": ROUTED["top_k"]}, "l1.moe")
        layers = [LayerSpec(norm("l0.n1"), learned, norm("l0.n2"), ffn("l0.ffn")),
                  LayerSpec(norm("l1.n1"), attn("l1.attn"), norm("l1.n2"), moe)]
        run = [RunEntry(0), RunEntry(1)]
    elif cfg.variant == "norms":
        # a layer that is a mixer alone; a layer with four norms, one of them on the stream itself (post-norm);
        # a layer that is a feed-forward alone and reads the stream without a norm
        layers = [LayerSpec(sub_blocks=[SubBlock("mixer", attn("l0.attn"), norm("l0.n1"))]),
                  LayerSpec(sub_blocks=[SubBlock("mixer", attn("l1.attn"), norm("l1.n1"), norm("l1.n1b"), after="branch"),
                                        SubBlock("ffn", ffn("l1.ffn"), norm("l1.n2"), norm("l1.n2s"), after="stream")]),
                  LayerSpec(sub_blocks=[SubBlock("ffn", ffn("l2.ffn"))])]
        run = [RunEntry(0), RunEntry(1), RunEntry(2)]
    elif cfg.variant == "reread":
        # the common block only, so that every run entry goes through the library's step executor: a layer that runs
        # twice, the second time reading the keys and values its first run wrote (it projects q alone)
        layers = [LayerSpec(norm("l0.n1"), attn("l0.attn"), norm("l0.n2"), ffn("l0.ffn")),
                  LayerSpec(norm("l1.n1"), attn("l1.attn"), norm("l1.n2"), ffn("l1.ffn"))]
        run = [RunEntry(0), RunEntry(1), RunEntry(0, cache_of=0)]
    else:   # "shared": a parallel block, a layer that runs twice, and a run that reads an earlier run's cache
        layers = [LayerSpec(norm("l0.n1"), attn("l0.attn"), norm("l0.n2"), ffn("l0.ffn"), arrangement="parallel"),
                  LayerSpec(norm("l1.n1"), attn("l1.attn"), norm("l1.n2"), ffn("l1.ffn"))]
        run = [RunEntry(0), RunEntry(1), RunEntry(1), RunEntry(0, cache_of=0)]
    return ModelSpec(cfg.architecture, D, cfg.vocab_size, 512,
                     PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": D}, "emb"),
                     layers, run, norm("final"), PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": D}, "emb"))


def toy_plain(raw, w, ids):
    """The toy architectures on whole sequences, from the plain parts."""
    D, H, Hkv, hd = raw["width"], raw["heads"], raw["kv_heads"], raw["head_dim"]
    eps = raw.get("eps", 1e-6)
    T = len(ids)
    pos = torch.arange(T)
    h = P.plain_embedding(torch.tensor(ids), w["emb.weight"])

    def qkv(p, x):
        q = P.plain_rope(P.plain_linear(x, w[p + ".q_proj.weight"]).reshape(T, H, hd), pos, 100.0)
        k = P.plain_rope(P.plain_linear(x, w[p + ".k_proj.weight"]).reshape(T, Hkv, hd), pos, 100.0)
        return q, k, P.plain_linear(x, w[p + ".v_proj.weight"]).reshape(T, Hkv, hd)

    def attn_out(p, q, k, v):
        return P.plain_linear(P.plain_attention(q, k, v, 1 / math.sqrt(hd)).reshape(T, H * hd), w[p + ".o_proj.weight"])

    def ffn(p, x):
        return P.plain_swiglu(x, w[p + ".gate_proj.weight"], w[p + ".up_proj.weight"], w[p + ".down_proj.weight"])

    def pre_norm_attn_layer(l, h):
        x = P.plain_rmsnorm(h, w[f"{l}.n1.weight"], eps)
        h = h + attn_out(f"{l}.attn", *qkv(f"{l}.attn", x))
        return h + ffn(f"{l}.ffn", P.plain_rmsnorm(h, w[f"{l}.n2.weight"], eps))

    if raw.get("variant") == "routed":
        # layer 0: attention whose q and k get a learned vector of their position added; layer 1: routed experts
        x = P.plain_rmsnorm(h, w["l0.n1.weight"], eps)
        q = P.plain_linear(x, w["l0.attn.q_proj.weight"]).reshape(T, H, hd) + w["l0.attn.pos.q_pos"][pos].unsqueeze(1)
        k = P.plain_linear(x, w["l0.attn.k_proj.weight"]).reshape(T, Hkv, hd) + w["l0.attn.pos.k_pos"][pos].unsqueeze(1)
        h = h + attn_out("l0.attn", q, k, P.plain_linear(x, w["l0.attn.v_proj.weight"]).reshape(T, Hkv, hd))
        h = h + ffn("l0.ffn", P.plain_rmsnorm(h, w["l0.n2.weight"], eps))
        x = P.plain_rmsnorm(h, w["l1.n1.weight"], eps)
        h = h + attn_out("l1.attn", *qkv("l1.attn", x))
        x = P.plain_rmsnorm(h, w["l1.n2.weight"], eps)
        logits = x @ w["l1.moe.router.weight"].t()
        order = logits.argsort(dim=-1, descending=True)
        kk = ROUTED["top_k"]
        out = torch.zeros_like(h)
        for t in range(T):
            chosen = order[t, :kk]
            weight = torch.softmax(logits[t, chosen], dim=0)
            for e, a in zip(chosen.tolist(), weight):
                up, down = w[f"l1.moe.experts.{e}.up.weight"], w[f"l1.moe.experts.{e}.down.weight"]
                out[t] += a * (torch.relu(x[t] @ up.t()) @ down.t())
        h = h + out
        # how far the last chosen expert's logit lies above the first one left out, relative to the largest logit
        sorted_logits = logits.gather(1, order)
        toy_plain.margin = (sorted_logits[:, kk - 1] - sorted_logits[:, kk]) / sorted_logits.abs().max(dim=1).values
    elif raw.get("variant") == "norms":
        rms = lambda v, name: P.plain_rmsnorm(v, w[name + ".weight"], eps)
        h = h + attn_out("l0.attn", *qkv("l0.attn", rms(h, "l0.n1")))                       # a mixer alone
        h = h + rms(attn_out("l1.attn", *qkv("l1.attn", rms(h, "l1.n1"))), "l1.n1b")       # a norm on the branch
        h = rms(h + ffn("l1.ffn", rms(h, "l1.n2")), "l1.n2s")                               # a norm on the stream
        h = h + ffn("l2.ffn", h)                                                            # no norm at all
    elif raw.get("variant", "state") == "state":
        x = P.plain_rmsnorm(h, w["l0.n1.weight"], eps)
        s, outs = torch.zeros(D), []
        for t in range(T):
            s = raw.get("decay", 0.5) * s + x[t]
            outs.append(s @ w["l0.toy.mix.weight"].t())
        h = h + torch.stack(outs)
        h = h + ffn("l0.ffn", P.plain_rmsnorm(h, w["l0.n2.weight"], eps))
        h = pre_norm_attn_layer("l1", h)
    elif raw.get("variant") == "reread":
        q0, k0, v0 = qkv("l0.attn", P.plain_rmsnorm(h, w["l0.n1.weight"], eps))
        h = h + attn_out("l0.attn", q0, k0, v0)
        h = h + ffn("l0.ffn", P.plain_rmsnorm(h, w["l0.n2.weight"], eps))
        h = pre_norm_attn_layer("l1", h)
        q2, _, _ = qkv("l0.attn", P.plain_rmsnorm(h, w["l0.n1.weight"], eps))       # keys and values of run entry 0
        h = h + attn_out("l0.attn", q2, k0, v0)
        h = h + ffn("l0.ffn", P.plain_rmsnorm(h, w["l0.n2.weight"], eps))
    else:
        x1, x2 = P.plain_rmsnorm(h, w["l0.n1.weight"], eps), P.plain_rmsnorm(h, w["l0.n2.weight"], eps)
        q0, k0, v0 = qkv("l0.attn", x1)
        h = h + attn_out("l0.attn", q0, k0, v0) + ffn("l0.ffn", x2)
        h = pre_norm_attn_layer("l1", h)
        h = pre_norm_attn_layer("l1", h)
        x1, x2 = P.plain_rmsnorm(h, w["l0.n1.weight"], eps), P.plain_rmsnorm(h, w["l0.n2.weight"], eps)
        q3, _, _ = qkv("l0.attn", x1)                     # keys and values are those of run entry 0
        h = h + attn_out("l0.attn", q3, k0, v0) + ffn("l0.ffn", x2)
    return P.plain_linear(P.plain_rmsnorm(h, w["final.weight"], eps), w["emb.weight"])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("variant", ["state", "shared", "routed", "norms", "reread"])
def test_toy_architecture_registered_from_the_test(tmp_path, variant, dtype):
    """Architectures made of the framework's parts and of parts defined in this file (a mixer with state of its own,
    a feed-forward with routing, a learned position encoding) and of other arrangements of a layer (a mixer alone,
    norms after a branch and on the stream, a feed-forward without a norm), registered from here and stepped in
    portions."""
    register_part("mixer", "toy_state", ToyStateMixer, replace=True)
    register_part("ffn", "toy_routed", ToyRoutedFFN, replace=True)
    register_part("position", "toy_learned", ToyLearnedPosition, replace=True)
    register_architecture("ToyForCausalLM", ToyConfig.from_dict, toy_spec, replace=True)
    raw = {"architectures": ["ToyForCausalLM"], "width": 48, "vocab": 211, "heads": 3, "kv_heads": 3, "head_dim": 16,
           "inner": 60, "decay": 0.7, "eps": 1e-5, "variant": variant}
    d = str(tmp_path / "toy")
    write_random_model(raw, 9, d, "float32" if dtype == "float32" else "bfloat16")
    cfg, w = P.read_model_dir(d)
    core = core_for(d, dtype, page=8, pages=40, max_seqs=3, max_tokens=256)
    layout = core.model.cache_layout
    if variant == "state":
        assert len(layout.state_planes) == 1 and layout.planes_per_group == [1]
    elif variant == "shared":
        assert layout.planes_per_group == [3] and not layout.refs[3].owns
    elif variant == "reread":
        assert layout.planes_per_group == [2] and not layout.refs[2].owns and all(core.runner.native.covers)
    rng = random.Random(10)
    seqs = {n: [rng.randrange(211) for _ in range(L)] for n, L in (("a", 50), ("b", 31), ("c", 44))}
    ref, sure = {}, {}
    for n, s in seqs.items():
        ref[n] = toy_plain(raw, w, s)
        sure[n] = torch.ones(len(s), dtype=torch.bool)
        if variant == "routed":
            # The experts sit in the last layer, so a token whose choice of experts is within rounding of a tie (either
            # choice is right) disturbs no other token; such tokens are left out of the comparison, and they are few.
            sure[n] = toy_plain.margin > (0.05 if dtype == "bfloat16" else 1e-4)
            assert float(sure[n].float().mean()) > 0.6
    fed = {n: 0 for n in seqs}
    toy_worst = 0.0
    core.open("a"), core.open("b")
    live, waiting = ["a", "b"], ["c"]          # "c" takes the slot (and its stale state) of whoever ends first
    while live:
        entries, exp = [], []
        for n in list(live):
            c = min(len(seqs[n]) - fed[n], rng.choice([1, 2, 7, 16]))
            entries.append(StepEntry(n, seqs[n][fed[n]: fed[n] + c], list(range(c))))
            exp.append((n, fed[n], c))
            fed[n] += c
        lg = core.step(entries).float().cpu()
        row = 0
        for n, at, c in exp:
            keep = sure[n][at: at + c]
            err = float((lg[row: row + c] - ref[n][at: at + c])[keep].abs().max()) if bool(keep.any()) else 0.0
            toy_worst = max(toy_worst, err)
            assert err <= atol_for("toy", dtype, ref), f"{variant} {dtype}: request {n} positions {at}..{at + c - 1}: {err}"
            row += c
            if fed[n] == len(seqs[n]):
                core.close(n)
                live.remove(n)
                if waiting:
                    core.open(waiting[0])
                    live.append(waiting.pop(0))
    record(f"toy {variant} {dtype}", toy_worst, logits_std(ref))
    core.cache.check()
