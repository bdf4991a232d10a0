"""Trace replay through bin/trace_run against the plain implementation: each request alone and
whole; most of it in one step and the last 32 tokens one by one; in portions of changing size
down to two tokens; and mixed, up to four live requests with so few pages that they are used
again.  In float32 and in bfloat16, on three tiny configurations."""
import os
import random
import tempfile

import pytest
import torch

from lightllm_b200.weights import write_random_model
from tests.plain.qwen2_plain import plain_forward, read_model_dir
from tests.tiny_configs import PAGE_SIZE, config
from tests.tolerances import atol_for, logits_std, record
from tests.trace_util import Trace, compare_with_plain, run_trace

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [5, 17, 33, 70, 101, 64, 49, 90], "B": [3, 9, 40, 70, 129, 200, 65, 96],
           "C": [4, 21, 47, 70, 150, 260, 80, 111], "D": [3, 40, 131, 300, 129, 700, 64, 257],
           "E": [2, 33, 130, 290, 128, 600, 65, 255]}


def make_sequences(name, seed):
    cfg = config(name)
    rng = random.Random(seed)
    return {f"r{i}": [rng.randrange(cfg["vocab_size"]) for _ in range(n)] for i, n in enumerate(LENGTHS[name])}


def build_trace(name):
    seqs = make_sequences(name, 11)
    # the same token sequences are replayed under new ids for each regime
    all_seqs, plan = {}, []
    for rid, toks in seqs.items():
        for regime in ("w", "t", "p"):
            all_seqs[f"{regime}{rid}"] = toks
    for rid, toks in seqs.items():
        all_seqs[f"m{rid}"] = toks
    tr = Trace(all_seqs)
    for rid in seqs:
        tr.whole(f"w{rid}")
    for rid, toks in seqs.items():
        if len(toks) > 2:
            tr.last_one_by_one(f"t{rid}")
    for i, rid in enumerate(seqs):
        tr.portions(f"p{rid}", [[16, 7, 2, 5, 3, 2], [2, 2, 9, 31, 4], [13, 2, 64, 3], [200, 33, 2, 129]][i % 4])
    single_max = tr.max_tokens
    mixed_ids = [f"m{rid}" for rid in seqs]
    prompt_len = {f"m{rid}": max(2, len(toks) - 12) if len(toks) > 14 else len(toks) for rid, toks in seqs.items()}
    tr.mixed(mixed_ids, prompt_len, seed=5, sizes=(2, 3, 7, 16, 40, 130) if name in "DE" else (2, 3, 5, 7, 16))
    return tr, seqs


@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_regimes(name, dtype, tmp_path):
    model_dir = str(tmp_path / "model")
    write_random_model(config(name), seed=3, out_dir=model_dir,
                       store_dtype="float32" if dtype == "float32" else "bfloat16")
    cfg, w = read_model_dir(model_dir)
    tr, seqs = build_trace(name)
    plain = {}
    for rid, toks in seqs.items():
        lg = plain_forward(cfg, w, toks)
        for regime in "wtpm":
            plain[f"{regime}{rid}"] = lg
    got = run_trace(model_dir, dtype, tr, str(tmp_path / "out"), ["--page-size", str(PAGE_SIZE[name])])
    once = {rid: plain[f"w{rid}"] for rid in seqs}
    std = logits_std(once)
    worst = compare_with_plain(tr, got, plain, atol_for(name, dtype, once), f"tiny {name} {dtype}")
    record(f"replay tiny {name} {dtype} ({len(tr.steps)} steps, pool for {tr.max_tokens} tokens)", worst, std)


def test_replay_default_page_size_and_float32_stored_weights_in_bfloat16(tmp_path):
    """A folder stored in float32 replayed with --dtype bfloat16 (tensors stored in 32 bits stay so),
    at trace_run's default page size."""
    model_dir = str(tmp_path / "model")
    write_random_model(config("B"), seed=4, out_dir=model_dir, store_dtype="float32")
    cfg, w = read_model_dir(model_dir)
    seqs = make_sequences("B", 12)
    tr = Trace({k: v for k, v in seqs.items()})
    for rid in list(seqs)[:4]:
        tr.portions(rid, [5, 2, 11])
    plain = {rid: plain_forward(cfg, w, toks) for rid, toks in seqs.items()}
    got = run_trace(model_dir, "bfloat16", tr, str(tmp_path / "out"))
    compare_with_plain(tr, got, plain, atol_for("B", "bfloat16", plain), "tiny B float32-stored bfloat16")
