"""The layers of a step through the library's step executor (csrc/step_executor.cu).

Launched kernel by kernel from the parts, a layer costs the host a chain of Python calls per launch (about 13 us each,
3 ms for a step of 24 layers), which sets the pace of every step that is not replayed from a CUDA graph.  Where
consecutive entries of the run list are the common block

    h += attention(rmsnorm(h));  h += gated_mlp(rmsnorm(h))          (src/engine/engine_server.cpp:1530-1880)

this module hands them to one call of the library, which issues the same kernels with the same choices as the parts
(the reference runs its layer loop in C++ too).  The model becomes an array of layer records when it is bound; a step
adds its metadata and the attention plans that the parts made for it.  Every other entry goes through the parts one
by one as before; what makes a layer fit is decided here from what the parts expose.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional

import torch

from ..csrc import ops
from ..parts import linear as L
from ..parts.attention import AttentionMixer
from ..parts.mlp import GatedMLP
from ..parts.norm import RMSNorm
from ..parts.rotary import NoPositionEncoding, RotaryEmbedding

MAX_GROUPS = 4
_P, _I, _F, _LL = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong


class NormDesc(ctypes.Structure):
    _fields_ = [("weight", _P), ("weight_dtype", _I), ("eps", _F)]


class AttentionDesc(ctypes.Structure):
    _fields_ = [("w_qkv", _P), ("b_qkv", _P), ("w_o", _P), ("b_o", _P), ("k_cache", _P), ("v_cache", _P), ("inv_freq", _P),
                ("num_slots", _LL), ("writes", _I), ("group", _I), ("num_heads", _I), ("num_kv_heads", _I), ("head_dim", _I),
                ("window", _I), ("scale", _F), ("rotary_dim", _I), ("interleaved", _I), ("plan", _I), ("freqs", _I), ("pad_", _I)]


class MlpDesc(ctypes.Structure):
    _fields_ = [("w_gate_up", _P), ("b_gate_up", _P), ("w_down", _P), ("b_down", _P), ("intermediate", _I), ("pad_", _I)]


class LayerDesc(ctypes.Structure):
    _fields_ = [("norm1", NormDesc), ("attn", AttentionDesc), ("norm2", NormDesc), ("mlp", MlpDesc)]


class ModelDesc(ctypes.Structure):
    _fields_ = [("layers", _P), ("num_layers", _I), ("hidden", _I), ("act_dtype", _I), ("num_sms", _I)]


class TileList(ctypes.Structure):
    _fields_ = [("span", _P), ("q0", _P), ("count", _I), ("bq", _I), ("nsplit", _I), ("pad_", _I)]


class AttentionPlan(ctypes.Structure):
    _fields_ = [("kind", _I), ("num_simt", _I), ("decode", TileList), ("items", TileList), ("item_k0", _P), ("item_nk", _P),
                ("item_part", _P), ("merge_span", _P), ("merge_q0", _P), ("merge_first", _P), ("merge_count", _P),
                ("num_parts", _I), ("num_merge", _I), ("simt", TileList * 2)]


class StepArgs(ctypes.Structure):
    _fields_ = [("token_ids", _P), ("positions", _P), ("span_row", _P), ("span_len", _P), ("span_pos", _P),
                ("block_tables", _P * MAX_GROUPS), ("slot_mapping", _P * MAX_GROUPS), ("residual", _P), ("workspace", _P),
                ("workspace_bytes", _LL), ("plans", _P), ("splitk_scratch", _P), ("splitk_floats", _LL),
                ("splitk_counters", _P), ("meet_counters", _P), ("error_flag", _P), ("stream", _P), ("splitk_tiles", _I),
                ("meet_counters_n", _I), ("T", _I), ("S", _I), ("max_pages", _I), ("page_size", _I), ("num_plans", _I),
                ("first_layer", _I), ("last_layer", _I), ("pad_", _I)]


_STRUCTS = (NormDesc, AttentionDesc, MlpDesc, LayerDesc, ModelDesc, TileList, AttentionPlan, StepArgs)


def _check_layout() -> None:
    sizes = (ctypes.c_int * len(_STRUCTS))()
    ops.lib().llb_step_struct_sizes(ctypes.addressof(sizes))
    for cls, n in zip(_STRUCTS, sizes):
        if ctypes.sizeof(cls) != n:
            raise ops.KernelError(f"step executor: {cls.__name__} is {ctypes.sizeof(cls)} bytes here and {n} in the library")


def _addr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _layer_record(block, view, dtype):
    """The record of one run of a layer and the tensors it points to, or None when the layer is of another kind."""
    if block.arrangement != "sequential" or len(block.subs) != 2 or view is None or view.k is None:
        return None
    a, f = block.subs
    if a.role != "mixer" or f.role != "ffn" or a.norm_after is not None or f.norm_after is not None:
        return None
    mixer, ffn, n1, n2 = a.part, f.part, a.norm_before, f.norm_before
    if type(mixer) is not AttentionMixer or type(ffn) is not GatedMLP or type(n1) is not RMSNorm or type(n2) is not RMSNorm:
        return None
    pos = mixer.position
    if type(pos) is RotaryEmbedding:
        inv_freq, rotary_dim, interleaved = pos.rotary_table()
        if rotary_dim <= 0 or inv_freq is None:
            return None
    elif type(pos) is NoPositionEncoding:
        inv_freq, rotary_dim, interleaved = None, 0, False
    else:
        return None
    weights = [mixer.w_qkv, mixer.w_o, ffn.w_gate_up, ffn.w_down, view.k, view.v]
    if any(w is None or w.dtype != dtype or not w.is_contiguous() for w in weights):
        return None                 # a tensor stored in another precision takes the parts' own paths
    if n1.out_dtype != dtype or n2.out_dtype != dtype or n1.hidden_size != mixer.hidden_size:
        return None
    if view.group is None or not 0 <= view.group < MAX_GROUPS:
        return None
    code = lambda t: ops.BF16 if t.dtype == torch.bfloat16 else ops.F32
    keep = weights + [mixer.b_qkv, mixer.b_o, ffn.b_gate_up, ffn.b_down, n1.weight, n2.weight, inv_freq]
    rec = LayerDesc()
    rec.norm1 = NormDesc(_addr(n1.weight), code(n1.weight), n1.eps)
    rec.norm2 = NormDesc(_addr(n2.weight), code(n2.weight), n2.eps)
    rec.attn = AttentionDesc(_addr(mixer.w_qkv), _addr(mixer.b_qkv), _addr(mixer.w_o), _addr(mixer.b_o), _addr(view.k),
                             _addr(view.v), _addr(inv_freq), view.k.shape[0], 1 if view.writes else 0, view.group,
                             mixer.num_heads, mixer.num_kv_heads, mixer.head_dim, mixer.window or 0, mixer.scale,
                             rotary_dim, 1 if interleaved else 0, 0, 0, 0)
    rec.mlp = MlpDesc(_addr(ffn.w_gate_up), _addr(ffn.b_gate_up), _addr(ffn.w_down), _addr(ffn.b_down),
                      ffn.intermediate_size, 0)
    freqs = None if inv_freq is None else (rotary_dim, bool(interleaved), pos.inv_freq_host.tobytes())
    return rec, keep, mixer, freqs


class NativeLayers:
    """The run entries that the library's step executor can run, and the call that runs a stretch of them."""

    def __init__(self, model, views, device):
        self.enabled = os.environ.get("LLB_NATIVE_STEP", "1") not in ("0", "")
        self.covers: List[bool] = [False] * len(model.run)
        self.calls = 0
        if not self.enabled or model.dtype not in (torch.bfloat16, torch.float32):
            return
        _check_layout()
        self.device = device
        self.dtype = model.dtype
        records, self._keep = [], []
        self._plan_keys: List[object] = []          # distinct attention plans of a step, by the mixers' prepare_key
        self._plan_mixer: List[AttentionMixer] = []
        hidden = None
        freq_sets: List[object] = []
        for i, entry in enumerate(model.run):
            made = _layer_record(model.layers[entry.layer], views[i], model.dtype)
            if made is not None:
                rec, keep, mixer, freqs = made
                key = mixer.prepare_key
                if key is None or (hidden is not None and mixer.hidden_size != hidden):
                    made = None
            if made is None:
                records.append(LayerDesc())
                continue
            hidden = mixer.hidden_size
            if key not in self._plan_keys:
                self._plan_keys.append(key)
                self._plan_mixer.append(mixer)
            rec.attn.plan = self._plan_keys.index(key)
            if freqs not in freq_sets:
                freq_sets.append(freqs)
            rec.attn.freqs = freq_sets.index(freqs)      # layers with the same frequencies share the step's rotary table
            records.append(rec)
            self._keep.append(keep)
            self.covers[i] = True
        if not any(self.covers):
            return
        self._records = (LayerDesc * len(records))(*records)
        self._model = ModelDesc(ctypes.addressof(self._records), len(records), hidden,
                                ops.BF16 if model.dtype == torch.bfloat16 else ops.F32, L.num_sms(device))
        self._plans = (AttentionPlan * len(self._plan_keys))()
        self._step = StepArgs()
        self._workspace: Optional[torch.Tensor] = None
        self._retired: List[torch.Tensor] = []          # workspaces that CUDA graphs captured earlier still use
        self._meet = ops.meet_counters(device)

    def stretch(self, i: int) -> int:
        """The end of the run entries from ``i`` on that one call can run (``i`` itself when entry ``i`` is not covered)."""
        j = i
        while j < len(self.covers) and self.covers[j]:
            j += 1
        return j

    # ------------------------------------------------------------------------------------------------------------------
    @staticmethod
    def _tiles(dst: TileList, tiles, bq: int, nsplit: int) -> None:
        span, q0, count = tiles
        dst.span, dst.q0, dst.count, dst.bq, dst.nsplit = span.data_ptr(), q0.data_ptr(), count, bq, nsplit

    def _fill_plan(self, dst: AttentionPlan, plan) -> None:
        ctypes.memset(ctypes.addressof(dst), 0, ctypes.sizeof(dst))
        if plan[0] in ("decode_mma", "decode_simt"):
            dst.kind = 0 if plan[0] == "decode_mma" else 1
            self._tiles(dst.decode, plan[1], 1, plan[2])
            return
        _, items, decode, simt = plan
        dst.kind = 2
        if items is not None:
            span, q0, count, cut = items
            self._tiles(dst.items, (span, q0, count), 128, 1)
            if cut is not None:
                k0, nk, part, parts, m_span, m_q0, m_first, m_count, n_merge = cut
                dst.item_k0, dst.item_nk, dst.item_part = k0.data_ptr(), nk.data_ptr(), part.data_ptr()
                dst.num_parts, dst.num_merge = parts, n_merge
                if n_merge:
                    dst.merge_span, dst.merge_q0 = m_span.data_ptr(), m_q0.data_ptr()
                    dst.merge_first, dst.merge_count = m_first.data_ptr(), m_count.data_ptr()
        if decode is not None:
            self._tiles(dst.decode, decode[0], 1, decode[1])
        if len(simt) > 2:
            raise ops.KernelError("step executor: an attention plan with more than two CUDA-core parts")
        dst.num_simt = len(simt)
        for n, (tiles, bq, nsplit) in enumerate(simt):
            self._tiles(dst.simt[n], tiles, bq, nsplit)

    def run(self, residual: torch.Tensor, ctx, first: int, last: int) -> None:
        """Run entries ``[first, last)`` (all covered) add into ``residual``."""
        lib = ops.lib()
        for n, mixer in enumerate(self._plan_mixer):
            self._fill_plan(self._plans[n], mixer._plan(ctx, self.dtype))
        s = self._step
        s.token_ids, s.positions = ctx.token_ids.data_ptr(), ctx.positions.data_ptr()
        s.span_row, s.span_len, s.span_pos = ctx.span_row.data_ptr(), ctx.span_len.data_ptr(), ctx.span_pos.data_ptr()
        if len(ctx.block_tables) > MAX_GROUPS:
            raise ops.KernelError(f"step executor: {len(ctx.block_tables)} cache groups; it carries {MAX_GROUPS}")
        for g, (bt, sm) in enumerate(zip(ctx.block_tables, ctx.slot_mapping)):
            s.block_tables[g], s.slot_mapping[g] = bt.data_ptr(), sm.data_ptr()
        s.residual = residual.data_ptr()
        s.plans, s.num_plans = ctypes.addressof(self._plans), len(self._plan_keys)
        sk = ops.splitk_scratch(self.device)
        if sk is not None:
            s.splitk_scratch, s.splitk_floats, s.splitk_counters, s.splitk_tiles = (sk[0].data_ptr(), sk[0].numel(),
                                                                                   sk[1].data_ptr(), sk[1].numel())
        else:
            s.splitk_scratch, s.splitk_floats, s.splitk_counters, s.splitk_tiles = None, 0, None, 0
        s.meet_counters, s.meet_counters_n = self._meet.data_ptr(), self._meet.numel()
        s.error_flag = ops.async_error_flag(self.device).data_ptr()
        s.stream = ops.current_stream()
        s.T, s.S, s.max_pages, s.page_size = ctx.T, ctx.num_spans, ctx.max_pages, ctx.page_size
        s.first_layer, s.last_layer = first, last
        s.workspace, s.workspace_bytes = None, 0
        need = lib.llb_step_workspace_need(ctypes.addressof(self._model), ctypes.addressof(s))
        if need < 0:
            raise ops.KernelError(lib.llb_last_error().decode("utf-8", "replace"))
        if self._workspace is None or self._workspace.numel() < need:
            if self._workspace is not None:
                self._retired.append(self._workspace)
            self._workspace = torch.empty(int(need * 1.25) + (1 << 20), dtype=torch.uint8, device=self.device)
        s.workspace, s.workspace_bytes = self._workspace.data_ptr(), self._workspace.numel()
        if lib.llb_step_layers(ctypes.addressof(self._model), ctypes.addressof(s)) != 0:
            raise ops.KernelError(lib.llb_last_error().decode("utf-8", "replace"))
        self.calls += 1
