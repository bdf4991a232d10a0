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
