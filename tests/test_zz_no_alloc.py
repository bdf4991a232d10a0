"""The entry point for callers that cannot allocate (llb_paged_attention_noalloc), called through
its exported C symbol, against the regular entry point that takes the scratch from the caller.

Some users of the kernel library may not call cudaMalloc where they run: a thread that launches
while another stream is being captured into a CUDA graph, a plug-in that lives on device pointers
an application handed to it, a loop that must never wait for the allocator.  For them split-KV
attention keeps its scratch in a fixed array inside the library.  This file checks that the two
entry points agree on two calls in a row (the second finds the first call's leftovers in the
array), and that a request beyond the array's size is refused with both numbers in the message.

It is collected last (see conftest.py), so a run that stops at the first failure has already run
every other test; it passes alone in a fresh process as well as after the others.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from lightllm_b200.csrc import build
    lib = ctypes.CDLL(build.library_path(build=True))
    lib.llb_last_error.restype = ctypes.c_char_p
    lib.llb_noalloc_scratch_floats.restype = ctypes.c_longlong
    lib.llb_attention_scratch_floats.restype = ctypes.c_longlong
    return lib


def _case(seed, lens, Hq, Hkv, hd, page, dtype, rows=1, bq=1):
    """One request per entry of ``lens`` (its context in keys), the last ``rows`` positions of each being the
    query rows of the step (decode-shaped with one row), cut into tiles of ``bq`` rows."""
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    pages_each = [-(-n // page) for n in lens]
    total = sum(pages_each) + 2
    perm = torch.randperm(total, generator=g).tolist()
    max_pages = max(pages_each)
    bt = torch.zeros((S, max_pages), dtype=torch.int32)
    for i, n in enumerate(pages_each):
        for lp in range(n):
            bt[i, lp] = perm.pop()
    kc = torch.randn((total * page, Hkv, hd), generator=g).to(dtype).to(dev)
    vc = torch.randn((total * page, Hkv, hd), generator=g).to(dtype).to(dev)
    q = torch.randn((S * rows, Hq * hd), generator=g).to(dtype).to(dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    tiles = [(i, q0) for i in range(S) for q0 in range(0, rows, bq)]
    return dict(q=q, kc=kc, vc=vc, bt=bt.to(dev), max_pages=max_pages, S=len(tiles), T=S * rows, bq=bq,
                tile_span=i32([t[0] for t in tiles]), tile_q0=i32([t[1] for t in tiles]),
                span_row=i32([i * rows for i in range(S)]), span_len=i32([rows] * S),
                span_pos=i32([n - rows for n in lens]))


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(lib, fn_name, c, out, Hq, Hkv, hd, page, nsplit, dtype_code, scratch=None):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [_ptr(c["q"]), _ptr(c["kc"]), _ptr(c["vc"]), _ptr(out), dtype_code, _ptr(c["tile_span"]),
            _ptr(c["tile_q0"]), c["S"], _ptr(c["span_row"]), _ptr(c["span_len"]), _ptr(c["span_pos"]), _ptr(c["bt"]),
            c["max_pages"], page, Hq, Hkv, hd, 0, ctypes.c_float(1.0 / math.sqrt(hd)), c["bq"], nsplit]
    if scratch is not None:
        args.append(_ptr(scratch))
    args.append(stream)
    return getattr(lib, fn_name)(*args)


@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, 0, 2e-5), (torch.bfloat16, 1, 2e-2)])
def test_noalloc_entry_matches_the_regular_one_on_two_calls_in_a_row(dtype, code, tol):
    lib = _library()
    Hq, Hkv, hd, page = 14, 2, 64, 16
    calls = [(_case(1, [700, 33, 257, 1], Hq, Hkv, hd, page, dtype), 8),
             (_case(2, [90, 1500], Hq, Hkv, hd, page, dtype), 5)]      # other sizes: the array holds leftovers
    for c, nsplit in calls:
        need = lib.llb_attention_scratch_floats(c["S"], Hq, hd, 1, nsplit)
        assert need <= lib.llb_noalloc_scratch_floats()
        scratch = torch.empty(need, dtype=torch.float32, device="cuda:0")
        want = torch.full((c["T"], Hq * hd), float("nan"), dtype=dtype, device="cuda:0")
        got = torch.full_like(want, float("nan"))
        assert _call(lib, "llb_paged_attention", c, want, Hq, Hkv, hd, page, nsplit, code, scratch) == 0, \
            lib.llb_last_error()
        assert _call(lib, "llb_paged_attention_noalloc", c, got, Hq, Hkv, hd, page, nsplit, code) == 0, \
            lib.llb_last_error()
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        assert torch.allclose(got.float(), want.float(), atol=tol, rtol=tol), \
            f"max diff {float((got.float() - want.float()).abs().max())}"


@pytest.mark.parametrize("dtype,code,tol", [(torch.float32, 0, 2e-5), (torch.bfloat16, 1, 2e-2)])
def test_noalloc_entry_with_tiles_of_several_rows(dtype, code, tol):
    """Portions of prompts (tiles of 4 rows) with their keys in 3 pieces: the general kernel through this entry."""
    lib = _library()
    Hq, Hkv, hd, page = 6, 2, 32, 8
    c = _case(4, [300, 41, 96], Hq, Hkv, hd, page, dtype, rows=10, bq=4)
    nsplit = 3
    need = lib.llb_attention_scratch_floats(c["S"], Hq, hd, 4, nsplit)
    assert need <= lib.llb_noalloc_scratch_floats()
    scratch = torch.empty(need, dtype=torch.float32, device="cuda:0")
    want = torch.full((c["T"], Hq * hd), float("nan"), dtype=dtype, device="cuda:0")
    got = torch.full_like(want, float("nan"))
    assert _call(lib, "llb_paged_attention", c, want, Hq, Hkv, hd, page, nsplit, code, scratch) == 0, lib.llb_last_error()
    assert _call(lib, "llb_paged_attention_noalloc", c, got, Hq, Hkv, hd, page, nsplit, code) == 0, lib.llb_last_error()
    torch.cuda.synchronize()
    assert not torch.isnan(got.float()).any()
    assert torch.allclose(got.float(), want.float(), atol=tol, rtol=tol)


def test_noalloc_entry_without_splits_has_no_size_limit():
    """With one piece per tile the array is never touched, so a tile list that would not fit in it is served."""
    lib = _library()
    Hq, Hkv, hd, page = 14, 2, 64, 16
    c = _case(5, [2200, 2300], Hq, Hkv, hd, page, torch.float32, rows=2048, bq=16)
    assert lib.llb_attention_scratch_floats(c["S"], Hq, hd, 16, 1) > lib.llb_noalloc_scratch_floats()
    want = torch.full((c["T"], Hq * hd), float("nan"), dtype=torch.float32, device="cuda:0")
    got = torch.full_like(want, float("nan"))
    assert _call(lib, "llb_paged_attention", c, want, Hq, Hkv, hd, page, 1, 0, torch.empty(1, device="cuda:0")) == 0, \
        lib.llb_last_error()
    assert _call(lib, "llb_paged_attention_noalloc", c, got, Hq, Hkv, hd, page, 1, 0) == 0, lib.llb_last_error()
    torch.cuda.synchronize()
    assert not torch.isnan(got).any()
    assert torch.allclose(got, want, atol=2e-5, rtol=2e-5)


def test_noalloc_entry_refuses_more_than_its_scratch_holds():
    lib = _library()
    Hq, Hkv, hd, page = 14, 2, 64, 16
    c = _case(3, [64] * 40, Hq, Hkv, hd, page, torch.float32)
    nsplit = 64
    need = lib.llb_attention_scratch_floats(c["S"], Hq, hd, 1, nsplit)
    assert need > lib.llb_noalloc_scratch_floats()
    out = torch.zeros((c["T"], Hq * hd), dtype=torch.float32, device="cuda:0")
    rc = _call(lib, "llb_paged_attention_noalloc", c, out, Hq, Hkv, hd, page, nsplit, 0)
    msg = lib.llb_last_error().decode()
    assert rc != 0 and str(need) in msg and str(lib.llb_noalloc_scratch_floats()) in msg
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0          # nothing was launched
