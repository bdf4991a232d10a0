"""The plain implementation checked against itself and against the reference's sampler (golden):
each part by an independent route (loops, float64), no GPU."""
import json
import math
import os

import numpy as np
import torch

from lightllm_b200.weights import write_random_model
from tests.plain import qwen2_plain as P
from tests.tiny_configs import config

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "sampling_golden.json")


def test_rmsnorm_rope_and_silu_by_loops():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(3, 10, generator=g, dtype=torch.float64)
    w = torch.randn(10, generator=g, dtype=torch.float64)
    y = P.plain_rmsnorm(x, w, 1e-5)
    for r in range(3):
        inv = 1.0 / math.sqrt(sum(float(v) ** 2 for v in x[r]) / 10 + 1e-5)
        for d in range(10):
            assert abs(float(y[r, d]) - float(x[r, d]) * inv * float(w[d])) < 1e-12
    q = torch.randn(4, 2, 8, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 5, 300])
    out = P.plain_rope(q, pos, 10000.0)
    assert torch.equal(out[0], q[0])                                       # position 0 is the identity
    for t in range(4):
        for i in range(4):
            inv_freq = np.float32(1.0 / 10000.0 ** (2 * i / 8))
            ang = float(np.float32(pos[t].item()) * inv_freq)
            a, b = float(q[t, 1, i]), float(q[t, 1, i + 4])
            assert abs(float(out[t, 1, i]) - (a * math.cos(ang) - b * math.sin(ang))) < 1e-6
            assert abs(float(out[t, 1, i + 4]) - (b * math.cos(ang) + a * math.sin(ang))) < 1e-6
    # rotation keeps the norm of every pair and only depends on relative position in q.k
    assert torch.allclose(out.norm(dim=-1), q.norm(dim=-1))
    inter = P.plain_rope(q, pos, 10000.0, interleaved=True)
    a, b = q[2, 0, 2], q[2, 0, 3]
    ang = float(np.float32(5.0) * np.float32(1.0 / 10000.0 ** (2 / 8)))
    assert abs(float(inter[2, 0, 2]) - float(a * math.cos(ang) - b * math.sin(ang))) < 1e-6
    part = P.plain_rope(q, pos, 10000.0, rotary_dim=4)
    assert torch.equal(part[..., 4:], q[..., 4:]) and not torch.equal(part[3, :, :4], q[3, :, :4])
    s = torch.tensor([-3.0, 0.0, 2.0], dtype=torch.float64)
    assert torch.allclose(P.plain_silu(s), s * torch.sigmoid(s))


def test_attention_by_loops_with_groups_and_window():
    g = torch.Generator().manual_seed(1)
    T, Hq, Hkv, hd = 9, 4, 2, 6
    q, k, v = (torch.randn(T, h, hd, generator=g, dtype=torch.float64) for h in (Hq, Hkv, Hkv))
    for window in (None, 3):
        out = P.plain_attention(q, k, v, 0.4, window)
        for i in range(T):
            for h in range(Hq):
                kh = h // 2
                js = [j for j in range(i + 1) if window is None or i - j < window]
                s = [float(q[i, h] @ k[j, kh]) * 0.4 for j in js]
                m = max(s)
                p = [math.exp(x - m) for x in s]
                ref = sum(pj * v[j, kh] for pj, j in zip(p, js)) / sum(p)
                assert torch.allclose(out[i, h], ref, atol=1e-12)
    assert torch.allclose(P.plain_attention(q, k, v, 0.4, 1), v.repeat_interleave(2, dim=1))   # window 1 sees itself only


def test_forward_is_causal_and_float32_agrees_with_float64(tmp_path):
    for name in "ABC":
        d = str(tmp_path / name)
        write_random_model(config(name), 2, d, "float32")
        cfg, w = P.read_model_dir(d)
        ids = [(7 * i + 3) % cfg["vocab_size"] for i in range(45)]
        l32 = P.plain_forward(cfg, w, ids, torch.float32)
        l64 = P.plain_forward(cfg, w, ids, torch.float64)
        assert float((l32.double() - l64).abs().max()) < 2e-5
        short = P.plain_forward(cfg, w, ids[:20], torch.float64)
        assert torch.allclose(short, l64[:20], atol=1e-12)                   # later tokens change nothing earlier
    # the window of tiny C matters: without it the late logits differ
    cfg2 = dict(cfg, use_sliding_window=False)
    assert float((P.plain_forward(cfg2, w, ids, torch.float64) - l64)[30:].abs().max()) > 1e-6
    assert torch.allclose(P.plain_forward(cfg2, w, ids, torch.float64)[:20], l64[:20], atol=1e-12)


def test_plain_sampler_against_the_reference_sampler():
    g = json.load(open(GOLDEN))
    logits = np.asarray(g["logits"], dtype=np.float32)
    for case in g["cases"]:
        hist = np.asarray(case["hist"], dtype=np.float64)
        if case["temperature"] < 1e-5:
            assert int(np.argmax(hist)) == int(np.argmax(logits)) and hist.max() == g["draws"]
            continue
        p = P.plain_sampling_probs(logits, case["temperature"], case["top_k"], case["top_p"], case["min_p"])
        assert set(np.nonzero(hist)[0]) <= set(np.nonzero(p)[0]), case
        freq = hist / g["draws"]
        sigma = np.sqrt(p * (1 - p) / g["draws"])
        assert np.all(np.abs(freq - p) <= 5 * sigma + 1e-4), case
    # the draw: first index whose cumulative mass reaches u
    p = np.array([0.0, 0.25, 0.0, 0.5, 0.25])
    assert [P.plain_draw(p, u) for u in (0.0, 0.2, 0.25, 0.26, 0.75, 0.76, 0.999)] == [1, 1, 1, 3, 3, 4, 4]


# ---------------------------------------------------------------------------------------------
# The plain attention and contraction against the reference's own CPU oracles
# ---------------------------------------------------------------------------------------------
ATTENTION_GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "attention_golden.json")


class _GoldenInputs:
    """The generator of tests/golden/golden_attention.cu (xorshift, 24 bits to a float in [-1, 1), times a scale in
    float32), so that the inputs need not be stored."""

    def __init__(self):
        self.state = 88172645463325252
        self.mask = (1 << 64) - 1

    def draw(self, n, scale):
        out = np.empty(n, dtype=np.float32)
        s = self.state
        for i in range(n):
            s ^= (s << 13) & self.mask
            s ^= s >> 7
            s ^= (s << 17) & self.mask
            out[i] = np.float32(((s >> 40) & 0xFFFFFF) / 8388608.0 - 1.0) * np.float32(scale)
        self.state = s
        return torch.from_numpy(out)


def test_plain_attention_and_head_agree_with_the_references_cpu_oracles():
    """``cpu_attention`` (tests/test_paged_attention_v2.cu:111-156: the query rows see every key),
    ``cpu_prefill_attention_causal`` (tests/test_paged_prefill.cu:164-215: the rows are the last positions, causal,
    ``acc / (l + 1e-8)``) and ``cpu_lm_head`` (tests/test_lm_head.cu:50-61), run once from the reference's own test
    programs (tests/golden/golden_attention.cu): grouped heads (``h // (Hq / Hkv)``), one kv head for all, the
    ``1 / sqrt(D)`` scale, the causal rule by absolute position and the ``x W^T`` head are theirs, not a reading."""
    with open(ATTENTION_GOLDEN) as f:
        golden = json.load(f)
    gen = _GoldenInputs()
    for case in golden["attention"]:
        T, Hq, Hkv, D, S = case["T"], case["Hq"], case["Hkv"], case["D"], case["seq_len"]
        q = gen.draw(T * Hq * D, 1.5).reshape(T, Hq, D)
        k = gen.draw(S * Hkv * D, 1.5).reshape(S, Hkv, D)
        v = gen.draw(S * Hkv * D, 1.0).reshape(S, Hkv, D)
        # the plain function takes whole sequences: the T query rows are the last T positions of S
        q_full = torch.zeros(S, Hq, D)
        q_full[S - T:] = q
        causal = P.plain_attention(q_full, k, v, 1.0 / math.sqrt(D))[S - T:]
        want = torch.tensor(case["causal"]).reshape(T, Hq, D)
        assert float((causal - want).abs().max()) < 2e-6, (T, Hq, Hkv, D, S)
        # every query row over every key is what the last position sees
        for t in range(T):
            q_last = torch.zeros(S, Hq, D)
            q_last[S - 1] = q[t]
            every = P.plain_attention(q_last, k, v, 1.0 / math.sqrt(D))[S - 1]
            want = torch.tensor(case["every_key"]).reshape(T, Hq, D)[t]
            assert float((every - want).abs().max()) < 2e-6, (T, Hq, Hkv, D, S, t)
    head = golden["lm_head"]
    hidden = gen.draw(head["D"], 1.0)
    embed = gen.draw(head["V"] * head["D"], 0.5).reshape(head["V"], head["D"])
    got = P.plain_linear(hidden[None, :], embed)[0]
    assert float((got - torch.tensor(head["logits"])).abs().max()) < 2e-6


def test_plain_norm_silu_and_embedding_agree_with_the_references_own_kernels():
    """``rms_norm`` (src/ops/norm.cu:11-75), ``silu`` (src/ops/elementwise.cu:27-33) and ``embedding``
    (src/ops/embedding.cu:9-30) of the reference, run once on a B200 from its own sources
    (tests/golden/golden_ops.cu, make_golden_gpu.sh); the inputs are drawn again here with the same generator."""
    with open(os.path.join(os.path.dirname(__file__), "golden", "ops_golden.json")) as f:
        golden = json.load(f)
    gen = _GoldenInputs()
    R, D = golden["rows"], golden["width"]
    x, w = gen.draw(R * D, 3.0).reshape(R, D), gen.draw(D, 1.0)
    want = torch.tensor(golden["rms_norm"]).reshape(R, D)
    assert float((P.plain_rmsnorm(x, w, golden["eps"]) - want).abs().max()) < 2e-6
    s = gen.draw(golden["silu_n"], 6.0)
    assert float((P.plain_silu(s) - torch.tensor(golden["silu"])).abs().max()) < 2e-6
    table = gen.draw(golden["vocab"] * golden["embed_width"], 1.0).reshape(golden["vocab"], golden["embed_width"])
    got = P.plain_embedding(torch.tensor(golden["ids"]), table)
    assert torch.equal(got, torch.tensor(golden["embedding"]).reshape(len(golden["ids"]), golden["embed_width"]))
