"""Decode steps through the persistent layer kernel (csrc/decode_layers.cu).

A step in which every request brings one token (at most 64 of them) spends its time in the chain of dependent
launches of a layer, not in the bytes it reads.  Where consecutive entries of the run list are the common block

    h += attention(rmsnorm(h));  h += gated_mlp(rmsnorm(h))          (src/engine/engine_server.cpp:1530-1880)

in bfloat16, with rotary (or no) positions and sizes the kernel takes, this module runs them as one kernel per
segment; every other entry, and every other kind of step, goes through the parts one by one as before.  What makes a
layer fit is decided here from what the parts expose; the parts do not know about it.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from ..csrc import ops
from ..parts import linear as L
from ..parts.attention import AttentionMixer
from ..parts.mlp import GatedMLP
from ..parts.norm import RMSNorm
from ..parts.rotary import NoPositionEncoding, RotaryEmbedding

MAX_ROWS = 64          # what the kernel takes
# Up to this many rows the persistent kernel is faster than the layers launched kernel by kernel (measured on B200 at
# the 0.5B sizes: 0.72 / 0.77 / 0.88 / 1.12 ms a step at 1 / 8 / 16 / 32 rows against 0.80 / 0.90 / 1.00 / 1.17; at 64 rows
# 1.66 against 1.54, where the attention's keys and the operands of 64 rows outweigh the saved launches).
DEFAULT_ROWS = 32
# The kernel pays where a layer is paced by its chain of stages, not by its bytes: up to this many bytes of weights a
# layer.  Measured: 30 MB a layer (0.5B sizes) 0.72 ms a step at one row against 0.80 launched kernel by kernel; 93 MB
# (1.5B) 1.36 against 1.33 at one row and 1.57 against 1.81 at eight; 404 MB (7B) 4.5 against 3.1: there the separate
# kernels stream their weights at 0.7 of the memory's bandwidth, which one block per multiprocessor walking through
# build, multiply and drain does not reach.
MAX_LAYER_BYTES = 128 << 20


def _layer_facts(block, view):
    """What the kernel needs of one run of a layer, or None when the layer is of another kind."""
    if block.arrangement != "sequential" or len(block.subs) != 2 or view is None:
        return None
    a, f = block.subs
    if a.role != "mixer" or f.role != "ffn" or a.norm_after is not None or f.norm_after is not None:
        return None
    mixer, ffn, n1, n2 = a.part, f.part, a.norm_before, f.norm_before
    if type(mixer) is not AttentionMixer or type(ffn) is not GatedMLP or type(n1) is not RMSNorm or type(n2) is not RMSNorm:
        return None
    pos = mixer.position
    if type(pos) is RotaryEmbedding:
        rotary = (pos.rotary_dim, pos.style == "interleaved", pos.theta)
    elif type(pos) is NoPositionEncoding:
        rotary = (0, False, 0.0)
    else:
        return None
    if (not view.writes or view.k is None or view.k.dtype != torch.bfloat16 or mixer.out_bias or ffn.bias
            or mixer.w_qkv is None or mixer.w_qkv.dtype != torch.bfloat16 or mixer.w_o.dtype != torch.bfloat16
            or ffn.w_gate_up.dtype != torch.bfloat16 or ffn.w_down.dtype != torch.bfloat16
            or n1.weight.dtype != n2.weight.dtype or n1.weight.dtype not in (torch.bfloat16, torch.float32)):
        return None
    sizes = (mixer.hidden_size, mixer.num_heads, mixer.num_kv_heads, mixer.head_dim, ffn.intermediate_size, rotary,
             mixer.scale)
    tensors = dict(w_qkv=mixer.w_qkv, w_o=mixer.w_o, w_gate_up=ffn.w_gate_up, w_down=ffn.w_down, b_qkv=mixer.b_qkv,
                   norm1_w=n1.weight, norm2_w=n2.weight, k_cache=view.k, v_cache=view.v, eps1=n1.eps, eps2=n2.eps,
                   window=mixer.window or 0, group=view.group)
    return sizes, tensors, pos


class Segment:
    """Consecutive run entries ``[begin, end)`` that one launch of the kernel runs."""

    def __init__(self, begin: int, end: int, sizes, layers, position, device):
        self.begin, self.end = begin, end
        (self.D, self.Hq, self.Hkv, self.hd, self.I, (self.rotary_dim, self.interleaved, _), self.scale) = sizes
        self.position = position
        self.windows = [d["window"] for d in layers]
        self.descriptors = ops.decode_layers_descriptors(layers, self.D, self.Hq, self.Hkv, self.hd, self.I, device)
        self.keep = layers                   # the descriptors hold addresses of these tensors
        self.counters = ops.decode_layers_counters(device)
        self.scratch: Optional[torch.Tensor] = None

    def splits(self, ctx) -> int:
        """Pieces of a request's keys: enough items for all multiprocessors, none shorter than 128 keys."""
        bound = ctx.max_pages * ctx.page_size              # the same for every step of this shape
        span = max(bound if w == 0 else min(bound, w) for w in self.windows)
        want = L.num_sms(ctx.device) // max(1, ctx.T * self.Hkv)
        return max(1, min(ops.MAX_FUSED_SPLITS, want, -(-span // 128)))

    def run(self, residual: torch.Tensor, ctx) -> None:
        nsplit = self.splits(ctx)
        need = ops.decode_layers_scratch_floats(MAX_ROWS, self.Hq, self.Hkv, self.hd, self.I, ops.MAX_FUSED_SPLITS)
        if self.scratch is None or self.scratch.numel() < need:
            self.scratch = torch.empty(need, dtype=torch.float32, device=residual.device)
        table = self.position.step_table(ctx) if self.rotary_dim else None
        ops.decode_layers(self.descriptors, self.end - self.begin, residual, self.D, self.Hq, self.Hkv, self.hd, self.I,
                          self.rotary_dim, self.interleaved, self.scale, table, ctx.span_pos, ctx.block_tables,
                          ctx.slot_mapping, ctx.max_pages, ctx.page_size, nsplit, self.scratch, self.counters)


class FusedDecode:
    """The segments of a model's run list that decode steps run through the persistent kernel."""

    def __init__(self, model, views, device):
        self.segments: List[Optional[Segment]] = [None] * len(model.run)      # by first run entry
        self.enabled = os.environ.get("LLB_FUSED_DECODE", "1") not in ("0", "")
        self.max_rows = min(MAX_ROWS, int(os.environ.get("LLB_FUSED_DECODE_MAX_ROWS", DEFAULT_ROWS)))
        if not self.enabled or model.dtype != torch.bfloat16 or not ops.has_tcgen05():
            self.enabled = False
            return
        facts = [_layer_facts(model.layers[e.layer], v) for e, v in zip(model.run, views)]
        groups = {f[1]["group"] for f in facts if f is not None}
        if any(g is None or g >= ops.MAX_FUSED_GROUPS for g in groups):
            facts = [None] * len(facts)
        i = 0
        while i < len(facts):
            if facts[i] is None or not self._sizes_ok(facts[i][0]) or self._layer_bytes(facts[i][1]) > MAX_LAYER_BYTES:
                i += 1
                continue
            j = i
            while j < len(facts) and facts[j] is not None and facts[j][0] == facts[i][0]:
                j += 1
            self.segments[i] = Segment(i, j, facts[i][0], [f[1] for f in facts[i:j]], facts[i][2], device)
            i = j
        self.enabled = any(s is not None for s in self.segments)

    @staticmethod
    def _layer_bytes(tensors) -> int:
        return sum(tensors[k].numel() * tensors[k].element_size() for k in ("w_qkv", "w_o", "w_gate_up", "w_down"))

    @staticmethod
    def _sizes_ok(sizes) -> bool:
        D, Hq, Hkv, hd, I, (rotary_dim, _, _), _ = sizes
        return ops.decode_layers_supports(1, D, Hq, Hkv, hd, I, rotary_dim)

    def takes(self, ctx) -> bool:
        # (one row a request: the kernel's attention stage makes a row's new key and value itself, beside the rows that
        # read the cache, so the rows of a step described row by row, which share requests, go kernel by kernel)
        return (self.enabled and ctx.decode_only and not ctx.rowwise and ctx.T <= self.max_rows
                and len(ctx.block_tables) <= ops.MAX_FUSED_GROUPS)

    def segment_at(self, run_index: int) -> Optional[Segment]:
        return self.segments[run_index]
