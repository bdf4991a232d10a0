"""A plain, slow implementation of the Qwen2 dense decoder: whole sequences, no cache, float32
(or float64) on the CPU, one function for each part.

It shares no code with the engine: it has its own safetensors reader, its own configuration
reading and its own formulas, written from the reference's files (cited per function; paths are
relative to the reference project).  The reference's whole model cannot be run on a machine
without a GPU (every tensor it touches is a CUDA tensor, src/tensor.cpp:62-72, and the build of
its engine needs the absent third_party/xgrammar), and its engine departs from the architecture
in known places, which are left out here on purpose: the q/k/v biases are added, every rotary
pair is rotated, a token sees its own key, and the output head follows ``tie_word_embeddings``.

What pins each formula to the reference's own code rather than to a reading of it
(tests/test_plain.py, golden files under tests/golden/ made by the scripts beside them):

* ``plain_attention``: the reference's CPU oracles ``cpu_attention`` (tests/test_paged_attention_v2.cu:111-156)
  and ``cpu_prefill_attention_causal`` (tests/test_paged_prefill.cu:164-215), compiled from its test
  programs: head grouping ``h // (Hq / Hkv)``, one kv head for all, the ``1/sqrt(D)`` scale, softmax,
  the causal rule by absolute position;
* ``plain_linear`` as the output head: ``cpu_lm_head`` (tests/test_lm_head.cu:50-61);
* ``plain_rmsnorm``, ``plain_silu``, ``plain_embedding``: the reference's own kernels ``rms_norm``,
  ``silu`` and ``embedding`` (src/ops/norm.cu, elementwise.cu, embedding.cu), run once on a B200;
* ``plain_sampling_probs`` / ``plain_draw``: the reference's ``sample()`` (src/ops/sampling.cpp);
* the rotation, the window rule, the q/k/v biases and the block's order of operations rest on the
  formulas cited at each function (the reference's rotation kernel turns one pair per head and its
  engine has no window), checked against loops and float64 in tests/test_plain.py.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

import numpy as np
import torch


# ---------------------------------------------------------------------------------------------
# Reading a model folder (format: src/model/model_loader.cpp:48-122)
# ---------------------------------------------------------------------------------------------
def read_safetensors(path: str) -> Dict[str, torch.Tensor]:
    """name -> float64/float32 CPU tensor (bf16 and f16 are widened exactly)."""
    with open(path, "rb") as f:
        data = f.read()
    (hlen,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + hlen].decode("utf-8"))
    base = 8 + hlen
    out: Dict[str, torch.Tensor] = {}
    for name, rec in header.items():
        if name == "__metadata__":
            continue
        b, e = rec["data_offsets"]
        raw = data[base + b: base + e]
        shape = rec["shape"]
        dt = rec["dtype"]
        if dt == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(np.float32)
        elif dt == "F16":
            arr = np.frombuffer(raw, dtype="<f2").astype(np.float32)
        elif dt == "BF16":
            u = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            arr = u.view(np.float32)
        elif dt == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"plain reader: dtype {dt} of {name}")
        out[name] = torch.from_numpy(arr.copy()).reshape(shape)
    return out


def read_model_dir(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(model_dir, "model.safetensors"))


# ---------------------------------------------------------------------------------------------
# Parts
# ---------------------------------------------------------------------------------------------
def plain_embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t,:] = table[id_t,:]  (src/ops/embedding.cu:9-18)."""
    return table[ids.long()]


def plain_rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """ss = sum x^2 (src/ops/norm.cu:19-23); inv = 1/sqrt(ss/D + eps) (:48-49); y = x*inv*w (:50-54)."""
    ss = (x * x).sum(dim=-1, keepdim=True)
    inv = 1.0 / torch.sqrt(ss / x.shape[-1] + eps)
    return x * inv * w


def plain_linear(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y = x W^T (+ b); W stored [out, in] (src/engine/engine_server.cpp:1542-1544, src/ops/gemm.cu:96-97)."""
    y = x @ w.t()
    return y if b is None else y + b


def plain_rope(x: torch.Tensor, positions: torch.Tensor, theta: float, rotary_dim: Optional[int] = None,
               interleaved: bool = False) -> torch.Tensor:
    """x [T, H, hd].  angle_i = pos * theta^(-2i/rotary_dim) (src/engine/engine_server.cpp:1570-1578);
    o_a = a cos - b sin, o_b = b cos + a sin over NeoX pairs (i, i + rotary_dim/2)
    (src/ops/rope.cu:54-59), on every pair (the reference's kernel rotates one, rope.cu:41-60).
    The inverse frequencies are float64 rounded to float32 and the angle is their float32
    product with the position, as the engine's documentation states."""
    T, H, hd = x.shape
    rd = hd if rotary_dim is None else rotary_dim
    half = rd // 2
    inv_freq = 1.0 / np.power(np.float64(theta), np.arange(0, rd, 2, dtype=np.float64) / rd)
    inv_freq = torch.from_numpy(inv_freq.astype(np.float32))
    ang = positions.to(torch.float32)[:, None] * inv_freq[None, :]          # float32 product
    cos, sin = torch.cos(ang).to(x.dtype)[:, None, :], torch.sin(ang).to(x.dtype)[:, None, :]
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:rd:2], x[..., 1:rd:2]
        out[..., 0:rd:2] = a * cos - b * sin
        out[..., 1:rd:2] = b * cos + a * sin
    else:
        a, b = x[..., :half], x[..., half:rd]
        out[..., :half] = a * cos - b * sin
        out[..., half:rd] = b * cos + a * sin
    return out


def plain_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                    window: Optional[int] = None) -> torch.Tensor:
    """q [T, Hq, hd], k, v [T, Hkv, hd] of one whole sequence -> [T, Hq, hd].
    kv_head = q_head / (Hq/Hkv) (src/kv_cache/paged_attention.cu:115); s = (q.k)*scale (:153-156);
    softmax over the visible keys (:158-163) and exactly acc/l; key j is visible to query i when
    j <= i (:1289-1291, with the token itself) and, with a window, i - j < window."""
    T, Hq, hd = q.shape
    Hkv = k.shape[1]
    group = Hq // Hkv
    out = torch.zeros_like(q)
    idx = torch.arange(T)
    visible = idx[None, :] <= idx[:, None]
    if window is not None:
        visible &= (idx[:, None] - idx[None, :]) < window
    for h in range(Hq):
        kh = h // group
        s = (q[:, h, :] @ k[:, kh, :].t()) * scale
        s = s.masked_fill(~visible, float("-inf"))
        m = s.max(dim=-1, keepdim=True).values
        p = torch.exp(s - m)
        out[:, h, :] = (p @ v[:, kh, :]) / p.sum(dim=-1, keepdim=True)
    return out


def plain_silu(x: torch.Tensor) -> torch.Tensor:
    """x / (1 + exp(-x))  (src/ops/elementwise.cu:27-33)."""
    return x / (1.0 + torch.exp(-x))


def plain_swiglu(x: torch.Tensor, wg: torch.Tensor, wu: torch.Tensor, wd: torch.Tensor) -> torch.Tensor:
    """(silu(x Wg^T) * (x Wu^T)) Wd^T  (src/engine/engine_server.cpp:1875-1880)."""
    return plain_linear(plain_silu(plain_linear(x, wg)) * plain_linear(x, wu), wd)


def layer_window(cfg: dict, layer: int) -> Optional[int]:
    if cfg.get("use_sliding_window", False) and layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"]):
        return cfg["sliding_window"]
    return None


def plain_block(h: torch.Tensor, positions: torch.Tensor, cfg: dict, w: Dict[str, torch.Tensor], layer: int) -> torch.Tensor:
    """One pre-norm block (src/engine/engine_server.cpp:1530-1880)."""
    p = f"model.layers.{layer}."
    Hq = cfg["num_attention_heads"]
    Hkv = cfg.get("num_key_value_heads", Hq)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // Hq
    eps = cfg.get("rms_norm_eps", 1e-6)
    T = h.shape[0]
    x = plain_rmsnorm(h, w[p + "input_layernorm.weight"], eps)
    q = plain_linear(x, w[p + "self_attn.q_proj.weight"], w.get(p + "self_attn.q_proj.bias")).reshape(T, Hq, hd)
    k = plain_linear(x, w[p + "self_attn.k_proj.weight"], w.get(p + "self_attn.k_proj.bias")).reshape(T, Hkv, hd)
    v = plain_linear(x, w[p + "self_attn.v_proj.weight"], w.get(p + "self_attn.v_proj.bias")).reshape(T, Hkv, hd)
    theta = cfg.get("rope_theta", 10000.0)
    q, k = plain_rope(q, positions, theta), plain_rope(k, positions, theta)
    a = plain_attention(q, k, v, 1.0 / math.sqrt(hd), layer_window(cfg, layer)).reshape(T, Hq * hd)
    h = h + plain_linear(a, w[p + "self_attn.o_proj.weight"])
    x = plain_rmsnorm(h, w[p + "post_attention_layernorm.weight"], eps)
    return h + plain_swiglu(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])


def plain_forward(cfg: dict, w: Dict[str, torch.Tensor], token_ids, dtype=torch.float32) -> torch.Tensor:
    """Logits [T, V] of one whole sequence (src/engine/engine_server.cpp:1526-1937, 2042)."""
    w = {k: (t.to(dtype) if t.is_floating_point() else t) for k, t in w.items()}
    ids = torch.as_tensor(list(token_ids), dtype=torch.long)
    positions = torch.arange(len(ids))
    h = plain_embedding(ids, w["model.embed_tokens.weight"])
    for layer in range(cfg["num_hidden_layers"]):
        h = plain_block(h, positions, cfg, w, layer)
    h = plain_rmsnorm(h, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return plain_linear(h, head)


def plain_greedy(cfg: dict, w: Dict[str, torch.Tensor], prompt: List[int], n_new: int, dtype=torch.float32) -> List[int]:
    """Greedy continuation, recomputing the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(n_new):
        logits = plain_forward(cfg, w, seq, dtype)
        nxt = int(torch.argmax(logits[-1]).item())
        out.append(nxt)
        seq.append(nxt)
    return out


# ---------------------------------------------------------------------------------------------
# Sampling (src/ops/sampling.cpp:22-335)
# ---------------------------------------------------------------------------------------------
def plain_sampling_probs(logits: np.ndarray, temperature: float, top_k: int = 0, top_p: float = 1.0,
                         min_p: float = 0.0) -> np.ndarray:
    """The distribution the sampler draws from: temperature (:81-84), top-k with ties kept
    (:91-137), softmax (:143-193), top-p prefix and renormalisation (:198-243), min-p and
    renormalisation (:248-278)."""
    x = logits.astype(np.float64) * (1.0 / max(temperature, 1e-8))
    V = x.shape[0]
    if 0 < top_k < V:
        kth = np.sort(x)[::-1][top_k - 1]
        x = np.where(x < kth, -np.inf, x)
    p = np.exp(x - x.max())
    p /= p.sum()
    if top_p < 1.0:
        order = np.argsort(-p, kind="stable")
        cum = np.cumsum(p[order])
        cutoff = int(np.searchsorted(cum, top_p, side="left")) + 1
        keep = np.zeros(V, dtype=bool)
        keep[order[:cutoff]] = True
        p = np.where(keep, p, 0.0)
        p /= p.sum()
    if min_p > 0.0:
        p = np.where(p < p.max() * min_p, 0.0, p)
        p /= p.sum()
    return p


def plain_draw(p: np.ndarray, u: float) -> int:
    """First index whose cumulative mass reaches u, skipping entries without mass (:284-334)."""
    cdf = np.cumsum(p)
    idx = int(np.searchsorted(cdf, u * cdf[-1], side="left"))
    idx = min(idx, len(p) - 1)
    while idx < len(p) - 1 and p[idx] == 0.0:
        idx += 1
    while p[idx] == 0.0 and idx > 0:
        idx -= 1
    return idx
