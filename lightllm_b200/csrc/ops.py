"""Python binding of the kernel library: thin, checked wrappers over its ``extern "C"`` entry points.

Every wrapper takes torch tensors that live on the GPU, checks dtype, shape and contiguity,
and launches on torch's current stream.  There is no fallback: if the library cannot be built
or loaded, or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
import re
from typing import Optional

import torch

from . import build as _build

F32, BF16 = 0, 1
EPI_STORE, EPI_STORE_F32, EPI_RESIDUAL, EPI_SWIGLU = 0, 1, 2, 3
ABI_VERSION = 21

_lib: Optional[ctypes.CDLL] = None


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    """The loaded kernel library (built on first use)."""
    global _lib
    if _lib is None:
        path = _build.library_path(build=True)
        try:
            handle = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"cannot load the kernel library {path}: {e}") from None
        _declare_signatures(handle)
        if handle.llb_abi_version() != ABI_VERSION:
            raise KernelError(f"{path} has ABI version {handle.llb_abi_version()}, expected {ABI_VERSION}")
        _lib = handle
    return _lib


_C_TYPES = {"int": ctypes.c_int, "float": ctypes.c_float, "long long": ctypes.c_longlong,
            "unsigned long long": ctypes.c_ulonglong, "cudaStream_t": ctypes.c_void_p, "const char*": ctypes.c_char_p}


def _declare_signatures(handle: ctypes.CDLL) -> None:
    """Argument and result types of every entry point, read from the ``LLB_EXPORT`` definitions in the
    sources the library was built from: pointers are passed as plain integers, without a ctypes
    object per argument."""
    pattern = re.compile(r"LLB_EXPORT\s+([\w\s\*]+?)\s*\b(llb_\w+)\s*\(([^)]*)\)\s*\{")

    def ctype(decl: str):
        decl = " ".join(decl.split())
        if decl == "void":
            return None
        if decl in _C_TYPES:
            return _C_TYPES[decl]
        if decl.endswith("*"):
            return ctypes.c_void_p
        raise KernelError(f"kernel library: no ctypes type for the C type {decl!r}")

    for name in _build.sources():
        with open(os.path.join(_build.CSRC_DIR, name)) as f:
            text = f.read()
        for ret, fn, args in pattern.findall(text):
            func = getattr(handle, fn)
            func.restype = ctype(ret)
            func.argtypes = [ctype(re.sub(r"\s*\w+$", "", a.strip())) for a in args.split(",") if a.strip() not in ("", "void")]


def _check(rc: int) -> None:
    if rc != 0:
        raise KernelError(lib().llb_last_error().decode("utf-8", "replace"))


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported dtype {t.dtype}; the kernels take float32 and bfloat16")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    """Device address of a tensor (None: a null pointer)."""
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("tensor is not on a CUDA device; there is no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"tensor of shape {tuple(t.shape)} must be contiguous")
    return t.data_ptr()


def _i32(t: Optional[torch.Tensor], what: str) -> Optional[int]:
    if t is not None and t.dtype != torch.int32:
        raise KernelError(f"{what} must be int32, got {t.dtype}")
    return _ptr(t)


_scoped_stream: Optional[int] = None


def torch_stream() -> "torch.cuda.Stream":
    """torch's current stream on the current device.  The device is named explicitly: asked without one,
    ``torch.cuda.current_stream()`` first looks for an available device type, which counts the devices through the
    driver every time (up to 0.14 ms a call on this machine, several calls a step)."""
    return torch.cuda.current_stream(torch.cuda.current_device())


class stream_scope:
    """Within the scope every launch goes to the stream that was current on entry, without asking torch
    again for each kernel.  The stream must not be switched inside the scope."""

    def __enter__(self):
        global _scoped_stream
        self._outer = _scoped_stream
        _scoped_stream = torch_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._outer
        return False


def _stream() -> int:
    s = _scoped_stream
    return s if s is not None else torch_stream().cuda_stream


def current_stream() -> int:
    """The stream that this module's launches go to right now (see :class:`stream_scope`)."""
    return _stream()


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor, err: Optional[torch.Tensor] = None) -> None:
    """out[t,:] = table[ids[t],:] as float.  ids int32 [T], table [V,D], out float32 [T,D]."""
    T, (V, D) = ids.numel(), table.shape
    if out.dtype != torch.float32 or tuple(out.shape) != (T, D):
        raise KernelError(f"embedding: out must be float32 [{T},{D}], got {out.dtype} {tuple(out.shape)}")
    _check(lib().llb_embedding(_i32(ids, "ids"), _ptr(table), _dt(table), _ptr(out), T, D, V,
                               _i32(err, "err"), _stream()))


def cast_add(src: torch.Tensor, dst: torch.Tensor, accumulate: bool = False) -> None:
    """dst = src (converted to dst's dtype), or dst += src with ``accumulate``; float32 or bfloat16 on either side."""
    if src.numel() != dst.numel():
        raise KernelError(f"cast_add: {tuple(src.shape)} does not fit {tuple(dst.shape)}")
    _check(lib().llb_cast_add(_ptr(src), _dt(src), _ptr(dst), _dt(dst), src.numel(), 1 if accumulate else 0, _stream()))


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r,:] = rmsnorm(x[rows[r],:]) * weight (rows = None: row r of x)."""
    D = x.shape[-1]
    R = rows.numel() if rows is not None else x.numel() // D
    if weight.numel() != D or out.numel() != R * D:
        raise KernelError(f"rmsnorm: sizes do not fit: x {tuple(x.shape)} weight {tuple(weight.shape)} out {tuple(out.shape)}")
    _check(lib().llb_rmsnorm(_ptr(x), _dt(x), _ptr(weight), _dt(weight), _ptr(out), _dt(out),
                             _i32(rows, "rows"), R, D, ctypes.c_float(eps), _stream()))


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int,
              out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None) -> None:
    """CUDA-core contraction a[M,K] @ w[N,K]^T with a fused epilogue (see EPI_*)."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: a is {tuple(a.shape)} but w is {tuple(w.shape)}")
    _check_epilogue_args(a, N, M, bias, epilogue, out, residual)
    _check(lib().llb_gemm_simt(_ptr(a), _dt(a), _ptr(w), _ptr(bias), _dt(w), _ptr(out), _ptr(residual),
                               epilogue, M, N, K, _stream()))


def _check_epilogue_args(a, N, M, bias, epilogue, out, residual) -> None:
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError(f"gemm: bias must be float32 [{N}], got {bias.dtype} {tuple(bias.shape)}")
    if epilogue == EPI_RESIDUAL:
        if residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N):
            raise KernelError(f"gemm: residual must be float32 [{M},{N}]")
        return
    want_shape = (M, N // 2) if epilogue == EPI_SWIGLU else (M, N)
    want_dtype = torch.float32 if epilogue == EPI_STORE_F32 else a.dtype
    if out is None or tuple(out.shape) != want_shape or out.dtype != want_dtype:
        got = None if out is None else (out.dtype, tuple(out.shape))
        raise KernelError(f"gemm: out must be {want_dtype} {want_shape}, got {got}")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: Optional[torch.Tensor],
                  inv_freq: Optional[torch.Tensor], rotary_dim: int, interleaved: bool, q_out: torch.Tensor,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Rotate q and k by position and write k, v rows into their cache slots.

    qkv [T, (Hq + 2*Hkv)*hd]; q_out [T, Hq*hd]; caches [slots, Hkv, hd].  Without caches
    (``k_cache is None``) only q is produced and qkv holds Hq heads only."""
    T = qkv.shape[0]
    write_kv = k_cache is not None
    hkv = num_kv_heads if write_kv else 0
    if qkv.shape[1] != (num_heads + 2 * hkv) * head_dim:
        raise KernelError(f"rope_kv_write: qkv has {qkv.shape[1]} columns, expected {(num_heads + 2 * hkv) * head_dim}")
    if q_out.dtype != qkv.dtype or q_out.numel() != T * num_heads * head_dim:
        raise KernelError("rope_kv_write: q_out does not fit")
    if write_kv and (k_cache.dtype != qkv.dtype or v_cache.dtype != qkv.dtype):
        raise KernelError("rope_kv_write: cache dtype differs from the activations'")
    if inv_freq is not None and (inv_freq.dtype != torch.float32 or inv_freq.numel() != rotary_dim // 2):
        raise KernelError("rope_kv_write: inv_freq must be float32 [rotary_dim/2]")
    _check(lib().llb_rope_kv_write(_ptr(qkv), _dt(qkv), _i32(positions, "positions"),
                                   _i32(slot_mapping, "slot_mapping"), _ptr(inv_freq), rotary_dim,
                                   1 if interleaved else 0, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
                                   T, num_heads, hkv, head_dim, 1 if write_kv else 0, _stream()))


def attention_smem_bytes(bq: int, group: int, head_dim: int) -> int:
    return int(lib().llb_attention_smem_bytes(bq, group, head_dim))


def attention_scratch_floats(num_tiles: int, num_heads: int, head_dim: int, bq: int, nsplit: int) -> int:
    return int(lib().llb_attention_scratch_floats(num_tiles, num_heads, head_dim, bq, nsplit))


def paged_attention_simt(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                         tile_span: torch.Tensor, tile_q0: torch.Tensor, num_tiles: int,
                         span_row: torch.Tensor, span_len: torch.Tensor, span_pos: torch.Tensor,
                         block_table: torch.Tensor, max_pages: int, page_size: int,
                         num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                         bq: int, nsplit: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """Attention of every query row of the listed tiles over its request's pages."""
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or out.dtype != q.dtype:
        raise KernelError("attention: q, caches and out must share a dtype")
    if nsplit > 1:
        need = attention_scratch_floats(num_tiles, num_heads, head_dim, bq, nsplit)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"attention: nsplit={nsplit} needs {need} floats of scratch")
    _check(lib().llb_paged_attention(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _dt(q),
        _i32(tile_span, "tile_span"), _i32(tile_q0, "tile_q0"), num_tiles,
        _i32(span_row, "span_row"), _i32(span_len, "span_len"), _i32(span_pos, "span_pos"),
        _i32(block_table, "block_table"), max_pages, page_size, num_heads, num_kv_heads, head_dim,
        window, ctypes.c_float(scale), bq, nsplit, _ptr(scratch), _stream()))


DEPI_STORE_F32, DEPI_RESIDUAL, DEPI_SWIGLU, DEPI_ROPE_KV = 1, 2, 3, 4


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, transposed: bool = False) -> torch.Tensor:
    """(cos, sin) of ``positions[t] * inv_freq[i]`` as float32 ``[T, len(inv_freq), 2]``, or pair-major
    ``[len(inv_freq), T, 2]`` with ``transposed``."""
    T, half = positions.numel(), inv_freq.numel()
    shape = (half, T, 2) if transposed else (T, half, 2)
    out = torch.empty(shape, dtype=torch.float32, device=positions.device)
    _check(lib().llb_rope_table(_i32(positions, "positions"), _ptr(inv_freq), _ptr(out), T, half,
                                1 if transposed else 0, _stream()))
    return out


_splitk = {}
_splitk_retired = []     # meeting places that a larger one replaced: CUDA graphs captured earlier still use them


def reserve_splitk_scratch(device: torch.device, floats: int, tiles: int) -> None:
    """Make sure the device has a zeroed meeting place of ``floats`` floats and ``tiles`` counters for
    split-K contractions with fused epilogues.  Call it when a model is bound, never inside a step.
    A meeting place that a larger one replaces is kept alive (and zero, as every launch leaves it): a graph
    captured while it was current goes on adding into it."""
    key = torch.device(device).index or 0
    have = _splitk.get(key)
    if have is None or have[0].numel() < floats or have[1].numel() < tiles:
        floats = max(floats, have[0].numel() if have else 0)
        tiles = max(tiles, have[1].numel() if have else 0)
        if have is not None:
            _splitk_retired.append(have)
        _splitk[key] = (torch.zeros(floats, dtype=torch.float32, device=device),
                        torch.zeros(tiles, dtype=torch.int32, device=device))


def splitk_scratch(device: torch.device):
    return _splitk.get(torch.device(device).index or 0)


def gemm_decode_supports(M: int, N: int, K: int, norm: bool, epilogue: int, head_dim: int = 0) -> bool:
    return bool(lib().llb_gemm_decode_supports(M, N, K, 1 if norm else 0, epilogue, head_dim))


def gemm_decode(w: torch.Tensor, epilogue: int, M: int, *, a: Optional[torch.Tensor] = None,
                x: Optional[torch.Tensor] = None, x_rows: Optional[torch.Tensor] = None,
                norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0, bias: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, split_k: int = 1,
                slot_mapping: Optional[torch.Tensor] = None,
                rope_table: Optional[torch.Tensor] = None, rotary_dim: int = 0, interleaved: bool = False,
                num_heads: int = 0, num_kv_heads: int = 0, head_dim: int = 0, q_out: Optional[torch.Tensor] = None,
                k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None) -> None:
    """The fused contraction of a step with at most 64 rows (see csrc/gemm_decode.cu).

    Operand: ``a`` [M, K] bf16, or the float rows ``x[x_rows]`` (``x[:M]`` without ``x_rows``) to be
    RMS-normalised with ``norm_weight`` and ``eps`` inside the kernel.  Epilogues: DEPI_STORE_F32
    (``out`` float [M, N]), DEPI_RESIDUAL (adds into ``residual``), DEPI_SWIGLU (``out`` bf16 [M, N/2]),
    DEPI_ROPE_KV (rotary by ``rope_table`` from :func:`rope_table`, ``q_out`` and the cache rows ``slot_mapping``)."""
    N, K = w.shape
    if w.dtype != torch.bfloat16:
        raise KernelError("gemm_decode takes bfloat16 weights")
    norm = x is not None
    if norm:
        if x.dtype != torch.float32 or x.shape[-1] != K or norm_weight is None or norm_weight.numel() != K:
            raise KernelError("gemm_decode: the normalised operand must be float32 [*, K] with a weight of K")
    elif a is None or a.dtype != torch.bfloat16 or tuple(a.shape) != (M, K):
        raise KernelError(f"gemm_decode: a must be bfloat16 [{M},{K}]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError(f"gemm_decode: bias must be float32 [{N}]")
    if epilogue == DEPI_RESIDUAL and (residual is None or residual.dtype != torch.float32 or tuple(residual.shape) != (M, N)):
        raise KernelError(f"gemm_decode: residual must be float32 [{M},{N}]")
    if epilogue == DEPI_STORE_F32 and (out is None or out.dtype != torch.float32 or tuple(out.shape) != (M, N)):
        raise KernelError(f"gemm_decode: out must be float32 [{M},{N}]")
    if epilogue == DEPI_SWIGLU and (out is None or out.dtype != torch.bfloat16 or tuple(out.shape) != (M, N // 2)):
        raise KernelError(f"gemm_decode: out must be bfloat16 [{M},{N // 2}]")
    if epilogue == DEPI_ROPE_KV:
        if q_out is None or q_out.dtype != torch.bfloat16 or q_out.numel() != M * num_heads * head_dim:
            raise KernelError("gemm_decode: q_out does not fit")
        if rotary_dim and (rope_table is None or rope_table.dtype != torch.float32
                           or rope_table.numel() != M * rotary_dim):
            raise KernelError("gemm_decode: rope_table must be float32 [M, rotary_dim/2, 2]")
        if slot_mapping is not None and (k_cache is None or v_cache is None or k_cache.dtype != torch.bfloat16):
            raise KernelError("gemm_decode: the cache must be bfloat16")
    scratch = splitk_scratch(w.device) if (split_k > 1 and epilogue in (DEPI_SWIGLU, DEPI_ROPE_KV)) else None
    if scratch is not None and scratch[1].numel() < -(-N // 128):
        scratch = None
    _check(lib().llb_gemm_decode(
        _ptr(w), _ptr(a), _ptr(x), _i32(x_rows, "x_rows"), _ptr(norm_weight),
        1 if (norm_weight is not None and norm_weight.dtype == torch.bfloat16) else 0, ctypes.c_float(eps),
        1 if norm else 0, _ptr(bias), _ptr(out), _ptr(residual), epilogue, M, N, K, split_k,
        _i32(slot_mapping, "slot_mapping"), _ptr(rope_table), rotary_dim,
        1 if interleaved else 0, num_heads, num_kv_heads, head_dim, _ptr(q_out), _ptr(k_cache), _ptr(v_cache),
        _ptr(scratch[0]) if scratch else ctypes.c_void_p(0), ctypes.c_longlong(scratch[0].numel() if scratch else 0),
        _ptr(scratch[1]) if scratch else ctypes.c_void_p(0), _ptr(async_error_flag(w.device)), _stream()))


def attention_tcgen05_supports(head_dim: int, page_size: int) -> bool:
    return bool(lib().llb_attention_tcgen05_supports(head_dim, page_size))


def paged_attention_tcgen05(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                            tile_span: torch.Tensor, tile_q0: torch.Tensor, num_tiles: int,
                            span_row: torch.Tensor, span_len: torch.Tensor, span_pos: torch.Tensor,
                            block_table: torch.Tensor, max_pages: int, page_size: int,
                            num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                            cut=None) -> None:
    """Tensor-core attention of the listed tiles (128 query rows each) over the requests' pages; bf16.

    ``cut`` = ``(tile_k0, tile_nk, tile_part, num_parts, merge_span, merge_q0, merge_first, merge_count,
    num_merge)`` cuts long key ranges into items (see ``StepContext.attention_items``); the partial results
    are merged by a second kernel."""
    for t in (q, k_cache, v_cache, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("attention_tcgen05 takes bfloat16 tensors")
    T = q.shape[0]
    num_slots = k_cache.shape[0]
    k0 = nk = part = scratch = None
    num_parts = 0
    if cut is not None:
        k0, nk, part, num_parts = cut[0], cut[1], cut[2], cut[3]
        if num_parts:
            scratch = torch.empty(num_parts * num_heads * 128 * (head_dim + 2), dtype=torch.float32, device=q.device)
    _check(lib().llb_paged_attention_tcgen05(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), T,
        _i32(tile_span, "tile_span"), _i32(tile_q0, "tile_q0"), num_tiles,
        _i32(span_row, "span_row"), _i32(span_len, "span_len"), _i32(span_pos, "span_pos"),
        _i32(block_table, "block_table"), max_pages, page_size, num_slots, num_heads, num_kv_heads, head_dim,
        window, ctypes.c_float(scale), _i32(k0, "tile_k0"), _i32(nk, "tile_nk"), _i32(part, "tile_part"),
        _ptr(scratch), num_parts, _ptr(async_error_flag(q.device)), _stream()))
    if cut is not None and num_parts:
        _check(lib().llb_attention_tcgen05_merge(
            _ptr(out), _i32(cut[4], "merge_span"), _i32(cut[5], "merge_q0"), _i32(cut[6], "merge_first"),
            _i32(cut[7], "merge_count"), cut[8], _i32(span_row, "span_row"), _i32(span_len, "span_len"),
            _ptr(scratch), num_parts, num_heads, head_dim, _stream()))


def paged_decode_mma_supports(num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return bool(lib().llb_paged_decode_mma_supports(num_heads, num_kv_heads, head_dim))


_cluster_splits: Optional[int] = None


_decode_resident = {}


def decode_mma_resident(head_dim: int) -> int:
    """Blocks of the decode attention kernel that one SM holds at a time for this head size."""
    n = _decode_resident.get(head_dim)
    if n is None:
        n = int(lib().llb_paged_decode_mma_resident(head_dim))
        if n <= 0:
            raise KernelError(lib().llb_last_error().decode("utf-8", "replace"))
        _decode_resident[head_dim] = n
    return n


def decode_mma_cluster_splits() -> int:
    """Up to this many splits the decode attention merges inside the kernel (a thread-block cluster); more
    need scratch and the merge kernel."""
    global _cluster_splits
    if _cluster_splits is None:
        _cluster_splits = int(lib().llb_paged_decode_mma_cluster_splits())
    return _cluster_splits


def paged_decode_mma(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, out: torch.Tensor,
                     tile_span: torch.Tensor, tile_q0: torch.Tensor, num_tiles: int, span_row: torch.Tensor,
                     span_pos: torch.Tensor, block_table: torch.Tensor, max_pages: int, page_size: int,
                     num_heads: int, num_kv_heads: int, head_dim: int, window: int, scale: float,
                     nsplit: int = 1, scratch: Optional[torch.Tensor] = None) -> None:
    """Tensor-core decode attention: one query row per tile over its request's pages; bf16.  ``nsplit`` cuts
    each request's keys; up to :func:`decode_mma_cluster_splits` the pieces are merged inside the kernel."""
    for t in (q, k_cache, v_cache, out):
        if t.dtype != torch.bfloat16:
            raise KernelError("paged_decode_mma takes bfloat16 tensors")
    if nsplit > decode_mma_cluster_splits():
        need = attention_scratch_floats(num_tiles, num_heads, head_dim, 1, nsplit)
        if scratch is None or scratch.dtype != torch.float32 or scratch.numel() < need:
            raise KernelError(f"decode attention: nsplit={nsplit} needs {need} floats of scratch")
    _check(lib().llb_paged_decode_mma(
        _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(out), _i32(tile_span, "tile_span"), _i32(tile_q0, "tile_q0"),
        num_tiles, _i32(span_row, "span_row"), _i32(span_pos, "span_pos"), _i32(block_table, "block_table"),
        max_pages, page_size, num_heads, num_kv_heads, head_dim, window, ctypes.c_float(scale), nsplit,
        _ptr(scratch), _stream()))


# Where the blocks that share a long row of logits meet (a 64-bit slot and a counter per row), per device.
_ARGMAX_ROWS = 4096
_argmax_scratch = {}


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    """out[r] = first index of the largest logit of row r.  logits float32 [R,V]."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1:
        raise KernelError("argmax: logits must be float32 with unit inner stride")
    if not logits.is_cuda:
        raise KernelError("argmax: logits are not on a CUDA device; there is no CPU path")
    key = logits.device.index or 0
    scratch = _argmax_scratch.get(key)
    if scratch is None:          # zero once: every launch leaves it zero
        scratch = _argmax_scratch[key] = torch.zeros(3 * _ARGMAX_ROWS, dtype=torch.int32, device=logits.device)
    _check(lib().llb_argmax(ctypes.c_void_p(logits.data_ptr()), R, V, ctypes.c_longlong(logits.stride(0)),
                            _i32(out, "out"), _ptr(scratch), _ARGMAX_ROWS, _stream()))


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: Optional[torch.Tensor],
           top_p: Optional[torch.Tensor], min_p: Optional[torch.Tensor], uniform: torch.Tensor,
           out: torch.Tensor) -> None:
    """One token per row from softmax(logits / temperature) after the top-k/top-p/min-p filters."""
    R, V = logits.shape
    if logits.dtype != torch.float32 or logits.stride(1) != 1 or not logits.is_cuda:
        raise KernelError("sample: logits must be float32 on a CUDA device with unit inner stride")
    for name, t in (("temperature", temperature), ("top_p", top_p), ("min_p", min_p), ("uniform", uniform)):
        if t is not None and (t.dtype != torch.float32 or t.numel() != R):
            raise KernelError(f"sample: {name} must be float32 [{R}]")
    _check(lib().llb_sample(ctypes.c_void_p(logits.data_ptr()), R, V, ctypes.c_longlong(logits.stride(0)),
                            _ptr(temperature), _i32(top_k, "top_k"), _ptr(top_p), _ptr(min_p), _ptr(uniform),
                            _i32(out, "out"), _stream()))


def launch_count() -> int:
    """Kernels this library has launched in this process."""
    return int(lib().llb_launch_count())


def has_tcgen05() -> bool:
    """Whether the library carries the tcgen05 tensor-core contraction."""
    return hasattr(lib(), "llb_gemm_tcgen05")


_async_err = {}


def async_error_flag(device: torch.device) -> torch.Tensor:
    """One int32 on the device that kernels with bounded waits raise when a wait ran out."""
    key = torch.device(device).index or 0
    t = _async_err.get(key)
    if t is None:
        t = _async_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return t


_reset_on_error = []      # counters that a kernel leaves in an unknown state when it gives up; cleared with the flag


def check_async_errors(device: torch.device) -> None:
    """Synchronises and raises if a kernel gave up on a wait (its output is then invalid)."""
    t = async_error_flag(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        for counters in _reset_on_error:
            if counters.device == t.device:
                counters.zero_()
        raise KernelError(f"a tensor-core kernel gave up waiting on a barrier (code {code}); its results are invalid")


# ---- the layers of a decode step as one persistent kernel (csrc/decode_layers.cu) -----------------------------------
MAX_FUSED_GROUPS = 4
MAX_FUSED_SPLITS = 32


def decode_layers_supports(M: int, D: int, Hq: int, Hkv: int, hd: int, I: int, rotary_dim: int) -> bool:
    return bool(lib().llb_decode_layers_supports(M, D, Hq, Hkv, hd, I, rotary_dim))


def decode_layers_descriptors(layers, D: int, Hq: int, Hkv: int, hd: int, I: int, device) -> torch.Tensor:
    """The device array of layer descriptors for :func:`decode_layers`.  ``layers``: one dict per layer with the
    tensors ``w_qkv``, ``w_o``, ``w_gate_up``, ``w_down``, ``b_qkv`` (or None), ``norm1_w``, ``norm2_w``, ``k_cache``,
    ``v_cache`` and the numbers ``eps1``, ``eps2``, ``window`` (0: none), ``group``.  The tensors must stay alive and
    in place as long as the descriptors are used."""
    import numpy as np
    size = int(lib().llb_decode_layers_desc_bytes())
    host = np.zeros(len(layers) * size, dtype=np.uint8)
    for i, d in enumerate(layers):
        for name in ("w_qkv", "w_o", "w_gate_up", "w_down"):
            if d[name].dtype != torch.bfloat16:
                raise KernelError(f"decode_layers: {name} must be bfloat16")
        if d["norm1_w"].dtype != d["norm2_w"].dtype or d["norm1_w"].dtype not in (torch.bfloat16, torch.float32):
            raise KernelError("decode_layers: the two norm weights must share a dtype (bfloat16 or float32)")
        if d["k_cache"].dtype != torch.bfloat16 or (d["b_qkv"] is not None and d["b_qkv"].dtype != torch.float32):
            raise KernelError("decode_layers: the cache must be bfloat16 and the bias float32")
        _check(lib().llb_decode_layers_describe(
            host.ctypes.data + i * size, _ptr(d["w_qkv"]), _ptr(d["w_o"]), _ptr(d["w_gate_up"]), _ptr(d["w_down"]),
            _ptr(d["b_qkv"]), _ptr(d["norm1_w"]), _ptr(d["norm2_w"]), 1 if d["norm1_w"].dtype == torch.bfloat16 else 0,
            ctypes.c_float(d["eps1"]), ctypes.c_float(d["eps2"]), _ptr(d["k_cache"]), _ptr(d["v_cache"]),
            int(d["window"] or 0), int(d["group"]), D, Hq, Hkv, hd, I))
    return torch.from_numpy(host).to(device)


def decode_layers_scratch_floats(M: int, Hq: int, Hkv: int, hd: int, I: int, nsplit: int) -> int:
    return int(lib().llb_decode_layers_scratch_floats(M, Hq, Hkv, hd, I, nsplit))


def decode_layers_counters(device) -> torch.Tensor:
    """The two counters on which the blocks of :func:`decode_layers` meet (zero between launches)."""
    t = torch.zeros(2, dtype=torch.int32, device=device)
    _reset_on_error.append(t)
    return t


def decode_layers(descriptors: torch.Tensor, num_layers: int, residual: torch.Tensor, D: int, Hq: int, Hkv: int, hd: int,
                  I: int, rotary_dim: int, interleaved: bool, scale: float, rope_table: Optional[torch.Tensor],
                  span_pos: torch.Tensor, block_tables, slot_mappings, max_pages: int, page_size: int, nsplit: int,
                  scratch: torch.Tensor, counters: torch.Tensor, timeline: Optional[torch.Tensor] = None,
                  timeline_block: int = 0) -> None:
    """All layers of a decode step (one token per request, at most 64) in one persistent kernel, in place on the
    float32 ``residual`` [M, D].  ``block_tables`` / ``slot_mappings``: one int32 tensor per cache group (up to 4).
    ``timeline`` (int64, 2 * (2 + 64 * layers) words) receives the milestones of block ``timeline_block`` as (label, SM cycle) pairs."""
    M = residual.shape[0]
    if residual.dtype != torch.float32 or tuple(residual.shape) != (M, D):
        raise KernelError(f"decode_layers: residual must be float32 [{M},{D}]")
    if len(block_tables) > MAX_FUSED_GROUPS or len(block_tables) != len(slot_mappings):
        raise KernelError(f"decode_layers: at most {MAX_FUSED_GROUPS} cache groups")
    bts = [_i32(t, "block_table") for t in block_tables] + [None] * (MAX_FUSED_GROUPS - len(block_tables))
    sms = [_i32(t, "slot_mapping") for t in slot_mappings] + [None] * (MAX_FUSED_GROUPS - len(slot_mappings))
    if scratch.dtype != torch.float32:
        raise KernelError("decode_layers: scratch must be float32")
    _check(lib().llb_decode_layers(
        _ptr(descriptors), num_layers, _ptr(residual), M, D, Hq, Hkv, hd, I, rotary_dim, 1 if interleaved else 0,
        ctypes.c_float(scale), _ptr(rope_table), _i32(span_pos, "span_pos"), *bts, *sms, max_pages, page_size, nsplit,
        _ptr(scratch), scratch.numel(), _ptr(counters), _ptr(async_error_flag(residual.device)), _ptr(timeline),
        timeline_block, _stream()))


def selftest_wait_expires(device: torch.device, limit_cycles: int = 1_000_000) -> torch.Tensor:
    """Run the library's self-test block whose waits nothing ever satisfies (csrc/selftest.cu): afterwards
    :func:`check_async_errors` raises.  Returns the two roles' outcomes (2 = left its wait unsatisfied)."""
    trace = torch.zeros(2, dtype=torch.int32, device=device)
    _check(lib().llb_selftest_wait_expires(_ptr(async_error_flag(device)), _ptr(trace), limit_cycles, _stream()))
    return trace


def selftest_mma_issue(device: torch.device, n: int = 64, a_tmem: bool = False, neighbours: int = 0, kind: int = 1,
                       iters: int = 256) -> dict:
    """The microbenchmark of csrc/selftest.cu: cycles that one thread needs to issue ``4 * iters`` tcgen05.mma of
    128 x n x 16 beside ``neighbours`` busy warps (kind 1: FMA chains, 2: softmax-like), and for the commit."""
    out = torch.zeros(4, dtype=torch.int64, device=device)
    _check(lib().llb_selftest_mma_issue(_ptr(out), n, int(a_tmem), neighbours, kind, iters, _stream()))
    issue, commit, arrive, _ = out.tolist()
    return {"cycles_per_mma": issue / (4 * iters), "commit_cycles": commit, "arrive_cycles": arrive}


_meet_counters = {}
_MEET_COUNTERS = 1 << 16


def meet_counters(device: torch.device) -> torch.Tensor:
    """The device's counters of wide split contractions (zero before and after every launch), made on first use."""
    key = torch.device(device).index or 0
    counters = _meet_counters.get(key)
    if counters is None:
        counters = _meet_counters[key] = torch.zeros(_MEET_COUNTERS, dtype=torch.int32, device=device)
    return counters


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], epilogue: int,
                 out: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None,
                 split_k: int = 1) -> None:
    """Tensor-core contraction a[M,K] @ w[N,K]^T (bf16, K a multiple of 8) with a fused epilogue.

    ``split_k`` > 1 cuts K into pieces that run as separate work items: up to 128 rows for the residual
    epilogue only (atomic adds); beyond, for every epilogue, through a meeting place in which the piece that
    arrives last adds all pieces in their order (the result does not depend on who arrives last)."""
    M, K = a.shape
    N, K2 = w.shape
    if K != K2:
        raise KernelError(f"gemm: a is {tuple(a.shape)} but w is {tuple(w.shape)}")
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        raise KernelError("gemm_tcgen05 takes bfloat16 operands")
    _check_epilogue_args(a, N, M, bias, epilogue, out, residual)
    partials = counters = None
    if split_k > 1 and M > 128:
        need = lib().llb_gemm_tcgen05_counters(M, N, split_k)
        if need > _MEET_COUNTERS:
            split_k = 1
        else:
            counters = meet_counters(a.device)
            partials = torch.empty(lib().llb_gemm_tcgen05_partial_floats(M, N, split_k), dtype=torch.float32,
                                   device=a.device)
    _check(lib().llb_gemm_tcgen05(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), _ptr(residual), epilogue, M, N, K,
                                  split_k, _ptr(partials), _ptr(counters), _ptr(async_error_flag(a.device)), _stream()))


def gemm_tcgen05_rope(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], rope_table: torch.Tensor,
                      slot_mapping: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor,
                      v_cache: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int = 64) -> None:
    """The q/k/v projection with heads of 64 or 128: a[M,K] @ w[N,K]^T, bias, NeoX rotation of the whole head by
    ``rope_table`` [hd/2, M, 2] (cos, sin; pair-major), q to ``q_out`` [M, Hq*hd], k and v to the cache rows
    ``slot_mapping`` [M] of ``k_cache`` / ``v_cache`` [slots, Hkv, hd] (a negative slot writes nothing)."""
    M, K = a.shape
    N, K2 = w.shape
    hd = head_dim
    if hd not in (64, 128) or K != K2 or N != (num_heads + 2 * num_kv_heads) * hd:
        raise KernelError(f"gemm_tcgen05_rope: a {tuple(a.shape)}, w {tuple(w.shape)}, heads {num_heads}/{num_kv_heads} of {hd}")
    for t, name in ((a, "a"), (w, "w"), (q_out, "q_out"), (k_cache, "k_cache"), (v_cache, "v_cache")):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise KernelError(f"gemm_tcgen05_rope: {name} must be contiguous bfloat16")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N):
        raise KernelError("gemm_tcgen05_rope: bias must be float32 of length N")
    if rope_table.dtype != torch.float32 or rope_table.numel() != M * hd or not rope_table.is_contiguous():
        raise KernelError("gemm_tcgen05_rope: rope_table must be float32 [hd/2, M, 2]")
    if slot_mapping.dtype != torch.int32 or slot_mapping.numel() != M:
        raise KernelError("gemm_tcgen05_rope: slot_mapping must be int32 [M]")
    if tuple(q_out.shape) != (M, num_heads * hd) or k_cache.shape[-1] != hd or k_cache.shape[-2] != num_kv_heads \
            or v_cache.shape != k_cache.shape:
        raise KernelError("gemm_tcgen05_rope: q_out must be [M, Hq*hd] and the caches [..., Hkv, hd]")
    _check(lib().llb_gemm_tcgen05_rope(_ptr(a), _ptr(w), _ptr(bias), M, N, K, _ptr(rope_table), _ptr(slot_mapping),
                                       _ptr(q_out), _ptr(k_cache), _ptr(v_cache), num_heads, num_kv_heads, hd,
                                       _ptr(async_error_flag(a.device)), _stream()))


def gemm_tcgen05_rope64(a, w, bias, rope_table, slot_mapping, q_out, k_cache, v_cache, num_heads, num_kv_heads) -> None:
    """:func:`gemm_tcgen05_rope` at heads of 64."""
    gemm_tcgen05_rope(a, w, bias, rope_table, slot_mapping, q_out, k_cache, v_cache, num_heads, num_kv_heads, 64)
