"""The attention mixer: grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from ..cache import CacheSpec, KVSpec
from ..config import PartSpec, part_class, register_part
from ..csrc import ops
from ..weights import WeightSpec
from . import linear as L
from .base import CacheView, LazyNorm, Mixer, Part

# Shared memory budget per block used to pick the tile height of the CUDA-core kernel.
_SMEM_BUDGET = 100 * 1024
_SMEM_LIMIT = 200 * 1024
# Portions of at least this many rows run on the tensor-core attention kernel (tiles of 128 rows, the rows beyond the
# portion masked): one block of the CUDA-core kernel walking a portion's keys takes hundreds of microseconds from a
# few hundred keys on, an item of the tensor-core kernel about two per 128 keys.
TENSOR_CORE_MIN_ROWS = 2
FUSED_ROPE_MAX_ROWS = 16
# Where the tensor-core kernels do not apply (float32, other head sizes): a portion of fewer than FEW_ROWS rows over
# MANY_KEYS keys or more is walked row by row with each row's keys in pieces, not by one block per tile of rows.
FEW_ROWS = 32
MANY_KEYS = 512
# Up to this many keys per request the decode attention's pieces are merged inside the kernel.
CLUSTER_MERGE_MAX_KEYS = 8192
# From this many rows on, heads of 64 or 128 get their rotation and cache write in the projection's tensor-core epilogue.
PREFILL_ROPE_MIN_ROWS = 16


class AttentionMixer(Mixer):
    """q, k, v projections (one fused contraction, bias in its epilogue), position encoding
    fused with the cache write, attention of every query over its request's pages, output
    projection added into the residual stream.

    Formulas: src/engine/engine_server.cpp:1542-1549 (projections), src/ops/rope.cu:54-59
    (rotation), src/kv_cache/paged_attention.cu:115,153-163 (grouping, scores, softmax),
    engine_server.cpp:1870-1871 (output projection and residual).  Unlike the reference the
    q/k/v biases are loaded and added, a token sees its own key, every portion is causal, and
    ``window`` limits a query to the latest ``window`` keys (itself included)."""

    graph_safe = True

    def __init__(self, prefix: str, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position: Optional[PartSpec] = None, qkv_bias: bool = True, out_bias: bool = False,
                 window: Optional[int] = None, scale: Optional[float] = None,
                 names: Optional[Dict[str, str]] = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} kv heads")
        self.prefix = prefix
        self.hidden_size, self.num_heads, self.num_kv_heads, self.head_dim = hidden_size, num_heads, num_kv_heads, head_dim
        self.qkv_bias, self.out_bias = qkv_bias, out_bias
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.names = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"}
        self.names.update(names or {})
        position = position or PartSpec("none")
        self.position = part_class("position", position.kind)(position.prefix, **position.params)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None

    def _n(self, which: str, what: str) -> str:
        return f"{self.prefix}.{self.names[which]}.{what}"

    def children(self):
        return [self.position]

    def cache_spec(self) -> CacheSpec:
        return CacheSpec(kv=KVSpec(self.num_kv_heads, self.head_dim, self.window))

    def weight_specs(self) -> List[WeightSpec]:
        D, hq, hkv = self.hidden_size, self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        specs = [WeightSpec(self._n("q", "weight"), (hq, D)), WeightSpec(self._n("k", "weight"), (hkv, D)),
                 WeightSpec(self._n("v", "weight"), (hkv, D)), WeightSpec(self._n("o", "weight"), (D, hq))]
        if self.qkv_bias:
            specs += [WeightSpec(self._n("q", "bias"), (hq,)), WeightSpec(self._n("k", "bias"), (hkv,)),
                      WeightSpec(self._n("v", "bias"), (hkv,))]
        if self.out_bias:
            specs.append(WeightSpec(self._n("o", "bias"), (D,)))
        return specs + self.position.weight_specs()

    def bind(self, tensors, dtype, device) -> None:
        ws = [tensors[self._n(p, "weight")] for p in "qkv"]
        wdt = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        self.w_qkv = torch.cat([w.to(wdt) for w in ws], dim=0).contiguous()
        self.w_o = tensors[self._n("o", "weight")]
        if self.qkv_bias:
            self.b_qkv = torch.cat([tensors[self._n(p, "bias")].float() for p in "qkv"]).contiguous()
        if self.out_bias:
            self.b_o = tensors[self._n("o", "bias")].float().contiguous()
        self.position.bind(tensors, dtype, device)
        L.reserve_fused_scratch(device, self.w_qkv.shape[0])

    # ------------------------------------------------------------------------------------------
    accepts_lazy_norm = True

    def _project_fused(self, x, ctx, cache: CacheView):
        """Norm (if still pending), q/k/v projection, bias, rotary positions and the cache write in one
        kernel, for steps of few rows in bfloat16.  Returns q, or None when the shape is not taken."""
        table = self.position.rotary_table()
        if table is None or self.w_qkv.dtype != torch.bfloat16 or not hasattr(self.position, "step_table"):
            return None
        if isinstance(x, LazyNorm) and not (x.fusable() is not None and x.num_rows <= L.FUSE_NORM_MAX_ROWS
                                           and self.w_qkv.shape[1] <= L.FUSE_NORM_MAX_COLS):
            x = x.materialize()
        lazy = isinstance(x, LazyNorm)
        rms = x.fusable() if lazy else None
        T = x.num_rows if lazy else x.shape[0]
        act_dtype = x.norm.out_dtype if lazy else x.dtype
        hq, hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        w = self.w_qkv if cache.writes else self.w_qkv[: hq * hd]
        # Beyond 16 rows the per-row loop of the rotary epilogue costs more than a separate rotation kernel
        # (measured at 64 rows: 25 us fused, 14 us apart).
        if T > FUSED_ROPE_MAX_ROWS or not L.decode_eligible(T, w, act_dtype, lazy, ops.DEPI_ROPE_KV, hd):
            return None
        b = self.b_qkv if (cache.writes or self.b_qkv is None) else self.b_qkv[: hq * hd]
        inv_freq, rotary_dim, interleaved = table
        q = torch.empty((T, hq * hd), dtype=torch.bfloat16, device=w.device)
        operand = dict(x=x.residual, norm_weight=rms[0], eps=rms[1]) if lazy else dict(a=x)
        ops.gemm_decode(w, ops.DEPI_ROPE_KV, T, bias=b, split_k=L.split_k_fused(T, w.shape[0], w.shape[1]),
                        slot_mapping=ctx.slot_mapping[cache.group] if cache.writes else None,
                        rope_table=self.position.step_table(ctx) if rotary_dim else None,
                        rotary_dim=rotary_dim, interleaved=interleaved, num_heads=hq, num_kv_heads=hkv, head_dim=hd,
                        q_out=q, k_cache=cache.k if cache.writes else None, v_cache=cache.v if cache.writes else None,
                        **operand)
        return q

    def _project_prefill_fused(self, x, ctx, cache: CacheView):
        """The projection of a long portion with bias, rotation and the cache write in the epilogue of the
        tensor-core kernel: bfloat16, heads of 64 or 128 rotated whole with NeoX pairs.  Returns q, or None."""
        T = x.shape[0]
        hd = self.head_dim
        table = self.position.rotary_table()
        if (T <= PREFILL_ROPE_MIN_ROWS or table is None or not cache.writes or hd not in (64, 128)
                or x.dtype != torch.bfloat16 or self.w_qkv.dtype != torch.bfloat16 or self.w_qkv.shape[1] % 8
                or not hasattr(self.position, "step_table")):
            return None
        _, rotary_dim, interleaved = table
        if rotary_dim != hd or interleaved:
            return None
        q = torch.empty((T, self.num_heads * hd), dtype=torch.bfloat16, device=x.device)
        ops.gemm_tcgen05_rope(x, self.w_qkv, self.b_qkv, self.position.step_table(ctx, transposed=True),
                              ctx.slot_mapping[cache.group], q, cache.k, cache.v, self.num_heads, self.num_kv_heads, hd)
        return q

    def forward(self, x, residual, ctx, cache: CacheView) -> None:
        q = self._project_fused(x, ctx, cache)
        if q is None:
            if isinstance(x, LazyNorm):
                x = x.materialize()
            q = self._project_prefill_fused(x, ctx, cache)
        if q is None:
            q = self._project(x, ctx, cache)
        attn = torch.empty_like(q)
        self.attend(q, cache, ctx, attn)
        L.linear(attn, self.w_o, self.b_o, L.RESIDUAL, residual=residual)

    def _project(self, x, ctx, cache: CacheView):
        T = x.shape[0]
        hq, hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        writes = cache.writes
        if writes:
            qkv = L.linear(x, self.w_qkv, self.b_qkv, L.STORE)
        else:  # the keys and values of another run entry are read; only q is projected
            qkv = L.linear(x, self.w_qkv[: hq * hd], None if self.b_qkv is None else self.b_qkv[: hq * hd], L.STORE)
        table = self.position.rotary_table()
        if table is None:
            table = (None, 0, False)
            qv = qkv[:, : hq * hd].reshape(T, hq, hd)
            kv = qkv[:, hq * hd: (hq + hkv) * hd].reshape(T, hkv, hd) if writes else None
            q2, k2 = self.position.apply(qv, kv, ctx.positions)
            if q2 is not qv:
                qkv[:, : hq * hd] = q2.reshape(T, hq * hd)
            if writes and k2 is not kv:
                qkv[:, hq * hd: (hq + hkv) * hd] = k2.reshape(T, hkv * hd)
        inv_freq, rotary_dim, interleaved = table
        q = torch.empty((T, hq * hd), dtype=x.dtype, device=x.device)
        ops.rope_kv_write(qkv, ctx.positions, ctx.slot_mapping[cache.group] if writes else None, inv_freq,
                          rotary_dim, interleaved, q, cache.k if writes else None, cache.v if writes else None,
                          hq, hkv, hd)
        return q

    def tile_height(self) -> int:
        group = self.num_heads // self.num_kv_heads
        for bq in (16, 8, 4, 2, 1):
            need = ops.attention_smem_bytes(bq, group, self.head_dim)
            if need <= _SMEM_BUDGET or (bq == 1 and need <= _SMEM_LIMIT):
                return bq
        raise ops.KernelError(
            f"attention with {group} query heads per kv head and head_dim {self.head_dim} does not fit "
            f"in shared memory even with one query row per block")

    def _plan(self, ctx, dtype):
        """Which kernels this step's attention takes and over which tiles: made once per step (in
        ``prepare`` when the engine runs it, so that the index arrays travel with the step's metadata)."""
        window = self.window or 0
        key = ("attention_plan", self.num_heads, self.num_kv_heads, self.head_dim, window, dtype)
        plan = ctx.memo.get(key)
        if plan is not None:
            return plan
        bf16 = dtype == torch.bfloat16
        if ctx.decode_only:
            S = ctx.num_spans
            bound = ctx.max_pages * ctx.page_size          # the same for every step of this shape
            span = bound if window == 0 else min(bound, window)
            want = max(1, -(-2 * L.num_sms(ctx.device) // (S * self.num_kv_heads)))       # blocks to fill the SMs twice
            nsplit = max(1, min(want, -(-span // 128)))
            mma = bf16 and ops.paged_decode_mma_supports(self.num_heads, self.num_kv_heads, self.head_dim)
            if mma and span <= CLUSTER_MERGE_MAX_KEYS:
                # Pieces that one thread-block cluster merges inside the kernel, which saves the merge kernel's
                # round trip: at most 8 (larger clusters start more slowly), and no more blocks than are resident
                # at once.
                resident = ops.decode_mma_resident(self.head_dim) * L.num_sms(ctx.device) // (S * self.num_kv_heads)
                nsplit = max(1, min(8, ops.decode_mma_cluster_splits(), resident, -(-span // 128)))
            plan = ("decode_mma" if mma else "decode_simt", ctx.tiles(1), nsplit)
        else:
            plan = self._plan_mixed(ctx, bf16, window)
        ctx.memo[key] = plan
        return plan

    def _plan_mixed(self, ctx, bf16: bool, window: int):
        """A step with portions of prompts, maybe beside decoded tokens.  Each span goes where its shape is served best:
        portions of two rows or more to the tensor-core kernel in tiles of 128 rows;
        single tokens to the decode kernel (its pieces along the keys merged in a cluster); the rest (everything in
        float32) to the CUDA-core kernel, in tiles of rows, or row by row with the keys in pieces for few rows over many
        keys."""
        tc_ok = bf16 and ops.attention_tcgen05_supports(self.head_dim, ctx.page_size)
        mma_ok = bf16 and ops.paged_decode_mma_supports(self.num_heads, self.num_kv_heads, self.head_dim)
        tensor, single, rows, rest = [], [], [], []
        rows_keys = 0
        for i, s in enumerate(ctx.spans):
            keys = s.start + s.length if window == 0 else min(s.start + s.length, window + s.length)
            if tc_ok and s.length >= TENSOR_CORE_MIN_ROWS:
                tensor.append(i)
            elif mma_ok and s.length == 1:
                single.append(i)
            elif s.length < FEW_ROWS and keys >= MANY_KEYS:
                rows.append(i)
                rows_keys = max(rows_keys, keys)
            else:
                rest.append(i)
        items = None
        if tensor:
            blocks_per_sm = 2 if self.head_dim <= 64 else 1
            items = ctx.attention_items(1, window, None, self.num_heads, blocks_per_sm * L.num_sms(ctx.device),
                                        select=tuple(tensor))
        decode = None
        if single:
            bound = ctx.max_pages * ctx.page_size
            span = bound if window == 0 else min(bound, window)
            resident = ops.decode_mma_resident(self.head_dim) * L.num_sms(ctx.device) // (len(single) * self.num_kv_heads)
            nsplit = max(1, min(8, ops.decode_mma_cluster_splits(), resident, -(-span // 128)))
            decode = (ctx.tiles(1, select=tuple(single)), nsplit)
        simt = []
        if rows:         # few rows over many keys: row by row, each row's keys in pieces
            simt.append((ctx.tiles(1, select=tuple(rows)), 1, max(2, min(16, -(-rows_keys // 256)))))
        if rest:
            bq = self.tile_height()
            simt.append((ctx.tiles(bq, select=tuple(rest)), bq, 1))
        return ("mixed", items, decode, simt)

    @property
    def prepare_key(self):
        """What the step's plan and rotary table depend on; attention layers that agree in it prepare once."""
        pos_key = ()
        if getattr(type(self.position), "prepare", None) is not Part.prepare:
            # a position encoding with a preparation of its own must say what it depends on, or runs every time
            pos_key = getattr(self.position, "prepare_key", None)
            if pos_key is None:
                return None
        return ("attention", self.num_heads, self.num_kv_heads, self.head_dim, self.window or 0, pos_key)

    def prepare(self, ctx, cache=None) -> None:
        self._plan(ctx, ctx.dtype)
        if hasattr(self.position, "prepare"):
            self.position.prepare(ctx)

    def attend(self, q, cache: CacheView, ctx, out) -> None:
        """out[t] = attention of query row t over positions <= its own (within the window)."""
        g = cache.group
        window = self.window or 0
        common = (ctx.span_row, ctx.span_len, ctx.span_pos, ctx.block_tables[g], ctx.max_pages, ctx.page_size,
                  self.num_heads, self.num_kv_heads, self.head_dim, window, self.scale)
        plan = self._plan(ctx, q.dtype)
        if plan[0] == "decode_mma":
            (tile_span, tile_q0, ntiles), nsplit = plan[1], plan[2]
            scratch = None
            if nsplit > ops.decode_mma_cluster_splits():
                scratch = torch.empty(ops.attention_scratch_floats(ntiles, self.num_heads, self.head_dim, 1, nsplit),
                                      dtype=torch.float32, device=q.device)
            ops.paged_decode_mma(q, cache.k, cache.v, out, tile_span, tile_q0, ntiles, ctx.span_row, ctx.span_pos,
                                 ctx.block_tables[g], ctx.max_pages, ctx.page_size, self.num_heads,
                                 self.num_kv_heads, self.head_dim, window, self.scale, nsplit, scratch)
        elif plan[0] == "decode_simt":
            self._simt(q, cache, out, plan[1], common, 1, plan[2])
        else:
            _, items, decode, simt = plan
            if items is not None:
                tile_span, tile_q0, ntiles, cut = items
                ops.paged_attention_tcgen05(q, cache.k, cache.v, out, tile_span, tile_q0, ntiles, *common, cut=cut)
            if decode is not None:
                (tile_span, tile_q0, ntiles), nsplit = decode
                ops.paged_decode_mma(q, cache.k, cache.v, out, tile_span, tile_q0, ntiles, ctx.span_row, ctx.span_pos,
                                     ctx.block_tables[g], ctx.max_pages, ctx.page_size, self.num_heads,
                                     self.num_kv_heads, self.head_dim, window, self.scale, nsplit, None)
            for tiles, bq, nsplit in simt:
                self._simt(q, cache, out, tiles, common, bq, nsplit)

    def _simt(self, q, cache, out, tiles, common, bq, nsplit) -> None:
        tile_span, tile_q0, ntiles = tiles
        scratch = None
        if nsplit > 1:
            scratch = torch.empty(ops.attention_scratch_floats(ntiles, self.num_heads, self.head_dim, bq, nsplit),
                                  dtype=torch.float32, device=q.device)
        ops.paged_attention_simt(q, cache.k, cache.v, out, tile_span, tile_q0, ntiles, *common, bq, nsplit, scratch)


register_part("mixer", "attention", AttentionMixer)
