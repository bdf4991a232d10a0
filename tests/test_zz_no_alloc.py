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


def _case(seed, lens, Hq, Hkv, hd, page, dtype):
    """Decode-shaped work: one query row per request over a paged context of ``lens`` keys."""
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
    q = torch.randn((S, Hq * hd), generator=g).to(dtype).to(dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    return dict(q=q, kc=kc, vc=vc, bt=bt.to(dev), max_pages=max_pages, S=S,
                tile_span=i32(list(range(S))), tile_q0=i32([0] * S), span_row=i32(list(range(S))),
                span_len=i32([1] * S), span_pos=i32([n - 1 for n in lens]))


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _call(lib, fn_name, c, out, Hq, Hkv, hd, page, nsplit, dtype_code, scratch=None):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [_ptr(c["q"]), _ptr(c["kc"]), _ptr(c["vc"]), _ptr(out), dtype_code, _ptr(c["tile_span"]),
            _ptr(c["tile_q0"]), c["S"], _ptr(c["span_row"]), _ptr(c["span_len"]), _ptr(c["span_pos"]), _ptr(c["bt"]),
            c["max_pages"], page, Hq, Hkv, hd, 0, ctypes.c_float(1.0 / math.sqrt(hd)), 1, nsplit]
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
        want = torch.full((c["S"], Hq * hd), float("nan"), dtype=dtype, device="cuda:0")
        got = torch.full_like(want, float("nan"))
        assert _call(lib, "llb_paged_attention", c, want, Hq, Hkv, hd, page, nsplit, code, scratch) == 0, \
            lib.llb_last_error()
        assert _call(lib, "llb_paged_attention_noalloc", c, got, Hq, Hkv, hd, page, nsplit, code) == 0, \
            lib.llb_last_error()
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any()
        assert torch.allclose(got.float(), want.float(), atol=tol, rtol=tol), \
            f"max diff {float((got.float() - want.float()).abs().max())}"


def test_noalloc_entry_refuses_more_than_its_scratch_holds():
    lib = _library()
    Hq, Hkv, hd, page = 14, 2, 64, 16
    c = _case(3, [64] * 40, Hq, Hkv, hd, page, torch.float32)
    nsplit = 64
    need = lib.llb_attention_scratch_floats(c["S"], Hq, hd, 1, nsplit)
    assert need > lib.llb_noalloc_scratch_floats()
    out = torch.zeros((c["S"], Hq * hd), dtype=torch.float32, device="cuda:0")
    rc = _call(lib, "llb_paged_attention_noalloc", c, out, Hq, Hkv, hd, page, nsplit, 0)
    msg = lib.llb_last_error().decode()
    assert rc != 0 and str(need) in msg and str(lib.llb_noalloc_scratch_floats()) in msg
    torch.cuda.synchronize()
    assert float(out.abs().max()) == 0.0          # nothing was launched
