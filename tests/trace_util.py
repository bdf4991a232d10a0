"""Building traces for bin/trace_run, running it, and comparing with the plain implementation."""
from __future__ import annotations

import json
import os
import random
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


def ceil64(n: int) -> int:
    return -(-n // 64) * 64


class Trace:
    """Steps for trace_run plus, for every wanted row, which request and position it is."""

    def __init__(self, sequences: Dict[str, List[int]]):
        self.sequences = sequences              # request id -> its full token sequence
        self.steps: List[dict] = []
        self.expect: Dict[int, List[Tuple[str, int]]] = {}
        self.fed: Dict[str, int] = {}
        self.live: Dict[str, int] = {}
        self.max_tokens = 0

    def step(self, feeds: Sequence[Tuple[str, int, Sequence[int]]], end: Sequence[str] = ()) -> None:
        """feeds: (request, number of next tokens, wanted places among them)."""
        n = len(self.steps)
        entries, exp = [], []
        for rid, count, want in feeds:
            at = self.fed.get(rid, 0)
            toks = self.sequences[rid][at: at + count]
            assert len(toks) == count and count > 0, (rid, at, count)
            entries.append({"id": rid, "tokens": toks, "want": list(want)})
            exp += [(rid, at + w) for w in want]
            self.fed[rid] = at + count
            self.live[rid] = at + count
        self.steps.append({"step": n, "entries": entries, "end": list(end)})
        if exp:
            self.expect[n] = exp
        self.max_tokens = max(self.max_tokens, sum(ceil64(v) for v in self.live.values()))
        for rid in end:
            self.live.pop(rid, None)

    # ---- the regimes -----------------------------------------------------------------------
    def whole(self, rid: str) -> None:
        n = len(self.sequences[rid])
        self.step([(rid, n, range(n))], end=[rid])

    def last_one_by_one(self, rid: str, tail: int = 32) -> None:
        n = len(self.sequences[rid])
        tail = min(tail, n - 1)
        self.step([(rid, n - tail, [n - tail - 1])])
        for i in range(tail):
            self.step([(rid, 1, [0])], end=[rid] if i == tail - 1 else [])

    def portions(self, rid: str, sizes: Sequence[int]) -> None:
        n = len(self.sequences[rid])
        at, i = 0, 0
        while at < n:
            c = min(sizes[i % len(sizes)], n - at)
            if n - at - c == 1:      # never leave a single token for a "portion"
                c += 1
            at += c
            i += 1
            self.step([(rid, c, range(c))], end=[rid] if at == n else [])

    def mixed(self, rids: Sequence[str], prompt_len: Dict[str, int], seed: int, max_live: int = 4,
              sizes: Sequence[int] = (2, 3, 5, 7, 16)) -> None:
        """Up to ``max_live`` requests at a time: portions of prompts (2..16 tokens) beside single
        decoded tokens; a request sometimes sits a step out; new ones start as others end."""
        rng = random.Random(seed)
        waiting = list(rids)
        live: List[str] = []
        while waiting or live:
            while waiting and len(live) < max_live:
                live.append(waiting.pop(0))
            feeds, end = [], []
            for rid in list(live):
                n = len(self.sequences[rid])
                at = self.fed.get(rid, 0)
                if len(live) > 1 and rng.random() < 0.2:
                    continue                                   # left out of this step
                if at < prompt_len[rid]:
                    c = min(rng.choice(list(sizes)), prompt_len[rid] - at)
                    if prompt_len[rid] - at - c == 1:
                        c += 1
                    feeds.append((rid, c, [c - 1] if rng.random() < 0.5 or at + c == prompt_len[rid] else []))
                else:
                    c = 1
                    feeds.append((rid, 1, [0]))
                if at + c == n:
                    end.append(rid)
                    live.remove(rid)
            if feeds:
                self.step(feeds, end)


def run_trace(model_dir: str, dtype: str, trace: Trace, out_dir: str, extra_args: Sequence[str] = (),
              env=None, max_tokens=None) -> Dict[int, np.ndarray]:
    """Run bin/trace_run on the trace, checking the ``done`` lines; returns step -> [wanted, vocab]."""
    cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
           "--max-tokens", str(max_tokens or trace.max_tokens), *extra_args]
    text = "".join(json.dumps(s) + "\n" for s in trace.steps)
    proc = subprocess.run(cmd, input=text, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env,
                          timeout=900)
    if proc.returncode != 0:
        raise AssertionError(f"trace_run exited with {proc.returncode}\nstderr:\n{proc.stderr[-4000:]}")
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {s['step']}" for s in trace.steps], proc.stdout[-2000:]
    with open(os.path.join(model_dir, "config.json")) as f:
        vocab = json.load(f)["vocab_size"]
    out = {}
    for n in trace.expect:
        arr = np.fromfile(os.path.join(out_dir, f"{n}.f32"), dtype="<f4")
        out[n] = arr.reshape(-1, vocab)
        assert out[n].shape[0] == len(trace.expect[n])
    unexpected = [f for f in os.listdir(out_dir) if f.endswith(".f32") and int(f[:-4]) not in trace.expect]
    assert not unexpected, f"files for steps in which nothing was wanted: {unexpected}"
    return out


def compare_with_plain(trace: Trace, got: Dict[int, np.ndarray], plain_logits: Dict[str, torch.Tensor],
                       atol: float, label: str = "") -> float:
    """Every wanted row against the plain implementation's logits of the whole sequence.
    On failure names the first wrong (step, request, position)."""
    worst = 0.0
    for n in sorted(trace.expect):
        for row, (rid, pos) in enumerate(trace.expect[n]):
            ref = plain_logits[rid][pos].numpy()
            err = float(np.max(np.abs(got[n][row] - ref)))
            worst = max(worst, err)
            if not err <= atol:
                raise AssertionError(
                    f"{label}: first wrong row at step {n}, request {rid!r}, position {pos}: max |diff| = {err:.3e} "
                    f"> {atol:.1e} (entries of the step: "
                    f"{[(e['id'], len(e['tokens'])) for e in trace.steps[n]['entries']]})")
    return worst
