"""Each kernel alone against a plain PyTorch float32 reference of the same op, at sizes other
than the engine's."""
import math

import numpy as np
import pytest
import torch

from tests.plain.qwen2_plain import (plain_attention, plain_draw, plain_rmsnorm, plain_rope, plain_sampling_probs,
                                     plain_silu)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from lightllm_b200.csrc import ops as o
    o.lib()
    return o


def dev():
    return torch.device("cuda:0")


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev())


DT = [torch.float32, torch.bfloat16]


@pytest.mark.parametrize("table_dtype", DT)
def test_embedding(ops, table_dtype):
    V, D = 301, 72
    table = rnd((V, D), table_dtype, 1)
    ids = torch.tensor([0, 300, 5, 5, 17, 123], dtype=torch.int32, device=dev())
    out = torch.empty((6, D), dtype=torch.float32, device=dev())
    err = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.embedding(ids, table, out, err)
    assert torch.equal(out, table.float()[ids.long()])
    assert int(err.item()) == 0
    bad = torch.tensor([1, V], dtype=torch.int32, device=dev())
    out2 = torch.empty((2, D), dtype=torch.float32, device=dev())
    ops.embedding(bad, table, out2, err)
    assert int(err.item()) == 1 and float(out2[1].abs().max()) == 0.0


@pytest.mark.parametrize("D", [24, 896, 1000, 1536, 5000])
@pytest.mark.parametrize("out_dtype", DT)
@pytest.mark.parametrize("w_dtype", DT)
def test_rmsnorm(ops, D, out_dtype, w_dtype):
    x = rnd((7, D), torch.float32, 2, 3.0)
    w = (1 + 0.1 * rnd((D,), torch.float32, 3)).to(w_dtype)
    for eps in (1e-6, 1e-2):
        out = torch.empty((7, D), dtype=out_dtype, device=dev())
        ops.rmsnorm(x, w, eps, out)
        ref = plain_rmsnorm(x.cpu(), w.float().cpu(), eps)
        tol = 1e-5 if out_dtype == torch.float32 else 2e-2
        assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=tol)
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=dev())
    out = torch.empty((3, D), dtype=out_dtype, device=dev())
    ops.rmsnorm(x, w, 1e-6, out, rows=rows)
    ref = plain_rmsnorm(x.cpu()[[6, 0, 3]], w.float().cpu(), 1e-6)
    assert torch.allclose(out.float().cpu(), ref, atol=2e-2 if out_dtype == torch.bfloat16 else 1e-5, rtol=2e-2)
    # many rows (widths that are multiples of 4 take the warp-per-row kernel from 8 rows on), also through a row list
    xm = rnd((61, D), torch.float32, 4, 3.0)
    out = torch.full((61, D), float("nan"), dtype=out_dtype, device=dev())
    ops.rmsnorm(xm, w, 1e-5, out)
    ref = plain_rmsnorm(xm.cpu(), w.float().cpu(), 1e-5)
    tol = 1e-5 if out_dtype == torch.float32 else 2e-2
    assert torch.allclose(out.float().cpu(), ref, atol=tol, rtol=tol)
    pick = torch.arange(60, -1, -3, dtype=torch.int32, device=dev())
    out = torch.full((pick.numel(), D), float("nan"), dtype=out_dtype, device=dev())
    ops.rmsnorm(xm, w, 1e-5, out, rows=pick)
    assert torch.allclose(out.float().cpu(), ref[pick.cpu().long()], atol=tol, rtol=tol)


GEMM_SHAPES = [(1, 50, 37), (3, 127, 172), (8, 64, 896), (9, 66, 45), (70, 130, 172), (129, 1000, 96), (5, 2, 8)]


def gemm_reference(a, w, bias, epi, residual):
    acc = a.double().cpu() @ w.double().cpu().t()
    if bias is not None:
        acc = acc + bias.double().cpu()
    if epi == 2:
        return residual.double().cpu() + acc
    if epi == 3:
        g, u = acc[:, 0::2], acc[:, 1::2]
        return plain_silu(g) * u
    return acc


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
@pytest.mark.parametrize("epi", [0, 1, 2, 3])
@pytest.mark.parametrize("dtypes", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                    (torch.bfloat16, torch.float32)])
def test_gemm_simt(ops, M, N, K, epi, dtypes):
    adt, wdt = dtypes
    a, w = rnd((M, K), adt, 4), rnd((N, K), wdt, 5, 0.2)
    if epi == 3 and N % 2:
        with pytest.raises(ops.KernelError, match="even N"):
            ops.gemm_simt(a, w, None, epi, torch.empty((M, N // 2), dtype=adt, device=dev()), None)
        return
    for bias in (None, rnd((N,), torch.float32, 6)):
        residual = rnd((M, N), torch.float32, 7)
        res0 = residual.clone()
        out = None
        if epi in (0, 3):
            out = torch.empty((M, N // 2 if epi == 3 else N), dtype=adt, device=dev())
        elif epi == 1:
            out = torch.empty((M, N), dtype=torch.float32, device=dev())
        ops.gemm_simt(a, w, bias, epi, out, residual if epi == 2 else None)
        ref = gemm_reference(a, w, bias, epi, res0)
        got = (residual if epi == 2 else out).double().cpu()
        exact_out = epi in (1, 2) or adt == torch.float32
        tol = 2e-5 * math.sqrt(K) if exact_out else 1e-2
        assert torch.allclose(got, ref, atol=tol * max(1.0, float(ref.abs().max())), rtol=0), \
            f"max diff {float((got - ref).abs().max())}"


TC_SHAPES = [(9, 50, 40), (16, 128, 64), (17, 130, 64), (33, 1152, 896), (64, 9728, 896), (65, 896, 4864),
             (128, 896, 896), (129, 200, 72), (300, 1000, 96), (2048, 1152, 896), (1000, 896, 4864), (12, 151936, 896),
             # many rows and features: tiles of 256 x 256 on pairs of CTAs (whole pairs, ragged edges, several rounds)
             (512, 2048, 64), (600, 2304, 136), (1000, 9728, 896), (4100, 2600, 200), (2048, 1536, 1536), (700, 1030, 264)]


@pytest.mark.parametrize("M,N,K", TC_SHAPES)
@pytest.mark.parametrize("epi", [0, 1, 2, 3])
def test_gemm_tcgen05(ops, M, N, K, epi):
    """The tensor-core contraction against float64 on the same bf16 operands."""
    if N > 100000 and epi != 1:
        pytest.skip("the vocabulary-sized case is the head's: float output only")
    a, w = rnd((M, K), torch.bfloat16, 40), rnd((N, K), torch.bfloat16, 41, 0.2)
    for bias, split_k in ((None, 1), (rnd((N,), torch.float32, 42), 1), (rnd((N,), torch.float32, 42), 5),
                          (None, 2)):
        if split_k > 1 and epi != 2 and M <= 128:
            continue        # few rows: only the residual epilogue can be split (atomic adds)
        residual = rnd((M, N), torch.float32, 43)
        res0 = residual.clone()
        out = None
        if epi in (0, 3):
            out = torch.full((M, N // 2 if epi == 3 else N), float("nan"), dtype=torch.bfloat16, device=dev())
        elif epi == 1:
            out = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
        ops.gemm_tcgen05(a, w, bias, epi, out, residual if epi == 2 else None, split_k)
        ops.check_async_errors(dev())
        ref = gemm_reference(a, w, bias, epi, res0)
        got = (residual if epi == 2 else out).double().cpu()
        assert not torch.isnan(got).any()
        tol = 1e-5 * math.sqrt(K) if epi in (1, 2) else 1e-2
        scale = max(1.0, float(ref.abs().max()))
        assert torch.allclose(got, ref, atol=tol * scale, rtol=0), f"max diff {float((got - ref).abs().max())}"
        if split_k > 1 and M > 128:
            # the pieces are added in their order, whoever arrives last: a second run gives the same bits,
            # and the meeting place's counters are zero again.  (A residual contraction without bias adds its pieces
            # straight into the residual instead: float adds in L2, equal up to the rounding of their order.)
            again = res0.clone() if epi == 2 else torch.empty_like(out)
            ops.gemm_tcgen05(a, w, bias, epi, None if epi == 2 else again, again if epi == 2 else None, split_k)
            if epi == 2 and bias is None:
                assert torch.allclose(again, residual, atol=2e-6 * scale, rtol=0)
            else:
                assert torch.equal(again, residual if epi == 2 else out)
            assert int(ops._meet_counters[dev().index or 0].abs().max()) == 0


DECODE_SHAPES = [(1, 1152, 896), (8, 9728, 896), (13, 896, 4864), (16, 130, 64), (17, 200, 136), (40, 1000, 96),
                 (64, 384, 192)]


@pytest.mark.parametrize("M,N,K", DECODE_SHAPES)
@pytest.mark.parametrize("norm", [False, True])
@pytest.mark.parametrize("epi", ["store_f32", "residual", "swiglu"])
def test_gemm_decode(ops, M, N, K, norm, epi):
    """The fused decode contraction: optional RMSNorm prologue, float / residual (split-K) / SwiGLU epilogues."""
    code = {"store_f32": ops.DEPI_STORE_F32, "residual": ops.DEPI_RESIDUAL, "swiglu": ops.DEPI_SWIGLU}[epi]
    if norm and not ops.gemm_decode_supports(M, N, K, norm, code):
        pytest.skip("the resident normalised operand does not fit in shared memory at this K")
    assert ops.gemm_decode_supports(M, N, K, norm, code)
    w = rnd((N, K), torch.bfloat16, 50, 0.2)
    bias = rnd((N,), torch.float32, 51)
    x = rnd((M + 3, K), torch.float32, 52, 2.0)
    nw = (1 + 0.1 * rnd((K,), torch.float32, 53))
    rows = torch.tensor([(5 * i + 2) % (M + 3) for i in range(M)], dtype=torch.int32, device=dev())
    if norm:
        a_ref = plain_rmsnorm(x.cpu()[rows.cpu().long()], nw.cpu(), 1e-5).to(torch.bfloat16)
        kw = dict(x=x, x_rows=rows, norm_weight=nw, eps=1e-5)
    else:
        a_ref = x[:M].to(torch.bfloat16).cpu()
        kw = dict(a=a_ref.to(dev()))
    ops.reserve_splitk_scratch(dev(), 64 * N, -(-N // 128))
    for split_k in ((1, 3) if epi in ("residual", "swiglu") else (1,)):
        residual = rnd((M, N), torch.float32, 54)
        res0 = residual.clone()
        out = None
        if epi == "store_f32":
            out = torch.full((M, N), float("nan"), dtype=torch.float32, device=dev())
        elif epi == "swiglu":
            out = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device=dev())
        ops.gemm_decode(w, code, M, bias=bias, out=out, residual=residual if epi == "residual" else None,
                        split_k=split_k, **kw)
        ops.check_async_errors(dev())
        ref = gemm_reference(a_ref, w, bias, {"store_f32": 1, "residual": 2, "swiglu": 3}[epi], res0)
        got = (residual if epi == "residual" else out).double().cpu()
        assert not torch.isnan(got).any()
        tol = (2e-2 if norm else 1e-5 * math.sqrt(K)) if epi != "swiglu" else 2e-2
        scale = max(1.0, float(ref.abs().max()))
        assert torch.allclose(got, ref, atol=tol * scale, rtol=0), f"max diff {float((got - ref).abs().max())}"


@pytest.mark.parametrize("M", [1, 8, 33])
@pytest.mark.parametrize("hd,rd,inter,Hq,Hkv", [(64, 64, False, 14, 2), (128, 64, True, 3, 1), (32, 32, False, 6, 3),
                                                (16, 16, False, 4, 2)])
@pytest.mark.parametrize("norm", [False, True])
def test_gemm_decode_rope_kv(ops, M, hd, rd, inter, Hq, Hkv, norm):
    """q/k/v projection with bias, rotary positions and the cache write in the epilogue, against the
    plain parts; and the q-only form that leaves the cache alone."""
    K, page, npages = 72, 8, 12
    N = (Hq + 2 * Hkv) * hd
    assert ops.gemm_decode_supports(M, N, K, norm, ops.DEPI_ROPE_KV, hd)
    w = rnd((N, K), torch.bfloat16, 60, 0.3)
    bias = rnd((N,), torch.float32, 61)
    x = rnd((M, K), torch.float32, 62, 2.0)
    nw = 1 + 0.1 * rnd((K,), torch.float32, 63)
    if norm:
        a_ref = plain_rmsnorm(x.cpu(), nw.cpu(), 1e-6).to(torch.bfloat16)
        kw = dict(x=x, norm_weight=nw.to(torch.bfloat16), eps=1e-6)
        a_ref = plain_rmsnorm(x.cpu(), nw.to(torch.bfloat16).float().cpu(), 1e-6).to(torch.bfloat16)
    else:
        a_ref = x.to(torch.bfloat16).cpu()
        kw = dict(a=a_ref.to(dev()))
    g = torch.Generator().manual_seed(64)
    pos = torch.randint(0, 3000, (M,), generator=g, dtype=torch.int32)
    slots = torch.randperm(npages * page, generator=g)[:M].to(torch.int32)
    if M > 2:
        slots[1] = -1
    theta = 10000.0
    inv = torch.from_numpy((1.0 / np.power(np.float64(theta), np.arange(0, rd, 2, dtype=np.float64) / rd))
                           .astype(np.float32)).to(dev())
    kc = torch.full((npages * page, Hkv, hd), 77.0, dtype=torch.bfloat16, device=dev())
    vc = torch.full((npages * page, Hkv, hd), 77.0, dtype=torch.bfloat16, device=dev())
    q = torch.full((M, Hq * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    table = ops.rope_table(pos.to(dev()), inv)
    ops.reserve_splitk_scratch(dev(), 64 * N, -(-N // 128))
    ops.gemm_decode(w, ops.DEPI_ROPE_KV, M, bias=bias, slot_mapping=slots.to(dev()), split_k=2 if M < 20 else 1,
                    rope_table=table, rotary_dim=rd, interleaved=inter, num_heads=Hq, num_kv_heads=Hkv, head_dim=hd,
                    q_out=q, k_cache=kc, v_cache=vc, **kw)
    ops.check_async_errors(dev())
    y = (a_ref.double() @ w.double().cpu().t() + bias.double().cpu()).float()
    qr = plain_rope(y[:, : Hq * hd].reshape(M, Hq, hd), pos, theta, rd, inter)
    kr = plain_rope(y[:, Hq * hd: (Hq + Hkv) * hd].reshape(M, Hkv, hd), pos, theta, rd, inter)
    vr = y[:, (Hq + Hkv) * hd:].reshape(M, Hkv, hd)
    tol = 3e-2
    scale = max(1.0, float(y.abs().max()))
    assert torch.allclose(q.float().cpu().reshape(M, Hq, hd), qr, atol=tol * scale, rtol=0)
    kexp = torch.full((npages * page, Hkv, hd), 77.0)
    vexp = kexp.clone()
    for t, sl in enumerate(slots.tolist()):
        if sl >= 0:
            kexp[sl], vexp[sl] = kr[t], vr[t]
    assert torch.allclose(kc.float().cpu(), kexp, atol=tol * scale, rtol=0)
    assert torch.allclose(vc.float().cpu(), vexp, atol=tol * scale, rtol=0)
    q2 = torch.full((M, Hq * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    kw2 = dict(kw)
    ops.gemm_decode(w[: Hq * hd], ops.DEPI_ROPE_KV, M, bias=bias[: Hq * hd].contiguous(),
                    rope_table=table, rotary_dim=rd, interleaved=inter, num_heads=Hq, num_kv_heads=Hkv, head_dim=hd,
                    q_out=q2, **kw2)
    ops.check_async_errors(dev())
    assert torch.allclose(q2.float(), q.float(), atol=tol * scale, rtol=0)
    sc = ops.splitk_scratch(dev())
    assert float(sc[0].abs().max()) == 0.0 and int(sc[1].abs().max()) == 0       # the meeting place is left clean

@pytest.mark.parametrize("M", [17, 64, 129, 300, 1000])
@pytest.mark.parametrize("Hq,Hkv,K,bias_on,hd", [(14, 2, 896, True, 64), (3, 1, 72, False, 64), (5, 5, 200, True, 64),
                                                 (12, 2, 1536, True, 128), (3, 1, 72, False, 128), (2, 2, 200, True, 128),
                                                 # 4,608 and 4,224 features: pair tiles of 256 x 256
                                                 (28, 4, 264, True, 128), (50, 8, 136, False, 64)])
def test_gemm_tcgen05_rope(ops, M, Hq, Hkv, K, bias_on, hd):
    """q/k/v projection of a long portion with bias, rotation and the cache write in the tensor-core
    epilogue, against the plain parts; heads of 64 (two heads a tile) and of 128 (the pairs' members lie in
    different halves of the tile)."""
    page = 16
    npages = -(-M // page) + 3
    N = (Hq + 2 * Hkv) * hd
    w = rnd((N, K), torch.bfloat16, 160, 0.3)
    bias = rnd((N,), torch.float32, 161) if bias_on else None
    a = rnd((M, K), torch.bfloat16, 162, 1.0)
    g = torch.Generator().manual_seed(164)
    pos = torch.randint(0, 30000, (M,), generator=g, dtype=torch.int32)
    slots = torch.randperm(npages * page, generator=g)[:M].to(torch.int32)
    slots[1] = -1
    slots[M - 2] = -1
    theta = 1000000.0
    inv = torch.from_numpy((1.0 / np.power(np.float64(theta), np.arange(0, hd, 2, dtype=np.float64) / hd))
                           .astype(np.float32)).to(dev())
    kc = torch.full((npages, page, Hkv, hd), 77.0, dtype=torch.bfloat16, device=dev())
    vc = torch.full((npages, page, Hkv, hd), 77.0, dtype=torch.bfloat16, device=dev())
    q = torch.full((M, Hq * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    table = ops.rope_table(pos.to(dev()), inv, transposed=True)
    assert torch.equal(table.transpose(0, 1), ops.rope_table(pos.to(dev()), inv))
    ops.gemm_tcgen05_rope(a, w, bias, table, slots.to(dev()), q, kc, vc, Hq, Hkv, hd)
    ops.check_async_errors(dev())
    y = a.double().cpu() @ w.double().cpu().t()
    if bias_on:
        y = y + bias.double().cpu()
    y = y.float()
    qr = plain_rope(y[:, : Hq * hd].reshape(M, Hq, hd), pos, theta, hd, False)
    kr = plain_rope(y[:, Hq * hd: (Hq + Hkv) * hd].reshape(M, Hkv, hd), pos, theta, hd, False)
    vr = y[:, (Hq + Hkv) * hd:].reshape(M, Hkv, hd)
    scale = max(1.0, float(y.abs().max()))
    tol = 2.0 ** -8 * scale      # one rounding to bfloat16 of a value of at most `scale`, and the table's float angles
    assert torch.allclose(q.float().cpu().reshape(M, Hq, hd), qr, atol=tol, rtol=0)
    kexp = torch.full((npages * page, Hkv, hd), 77.0)
    vexp = kexp.clone()
    for t, sl in enumerate(slots.tolist()):
        if sl >= 0:
            kexp[sl], vexp[sl] = kr[t], vr[t]
    assert torch.allclose(kc.float().cpu().reshape(-1, Hkv, hd), kexp, atol=tol, rtol=0)
    assert torch.allclose(vc.float().cpu().reshape(-1, Hkv, hd), vexp, atol=tol, rtol=0)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("hd,rd,inter", [(16, 16, False), (32, 32, True), (64, 64, False), (48, 32, False),
                                         (128, 64, True)])
def test_rope_kv_write(ops, dtype, hd, rd, inter):
    T, Hq, Hkv, page, npages = 11, 3, 1, 8, 6
    qkv = rnd((T, (Hq + 2 * Hkv) * hd), dtype, 8)
    pos = torch.tensor([0, 1, 2, 40, 41, 7, 100, 3000, 5, 6, 7], dtype=torch.int32, device=dev())
    slots = torch.tensor([3, 9, 47, 0, 1, 2, 21, 22, 8, -1, 30], dtype=torch.int32, device=dev())
    theta = 10000.0
    inv = torch.from_numpy((1.0 / np.power(np.float64(theta), np.arange(0, rd, 2, dtype=np.float64) / rd))
                           .astype(np.float32)).to(dev())
    kc = torch.full((npages * page, Hkv, hd), 77.0, dtype=dtype, device=dev())
    vc = torch.full((npages * page, Hkv, hd), 77.0, dtype=dtype, device=dev())
    q = torch.empty((T, Hq * hd), dtype=dtype, device=dev())
    ops.rope_kv_write(qkv, pos, slots, inv, rd, inter, q, kc, vc, Hq, Hkv, hd)
    x = qkv.float().cpu()
    qr = plain_rope(x[:, : Hq * hd].reshape(T, Hq, hd), pos.cpu(), theta, rd, inter)
    kr = plain_rope(x[:, Hq * hd: (Hq + Hkv) * hd].reshape(T, Hkv, hd), pos.cpu(), theta, rd, inter)
    vr = x[:, (Hq + Hkv) * hd:].reshape(T, Hkv, hd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(q.float().cpu().reshape(T, Hq, hd), qr, atol=tol, rtol=tol)
    kexp = torch.full((npages * page, Hkv, hd), 77.0)
    vexp = kexp.clone()
    for t, s in enumerate(slots.tolist()):
        if s >= 0:
            kexp[s], vexp[s] = kr[t], vr[t]
    assert torch.allclose(kc.float().cpu(), kexp, atol=tol, rtol=tol)
    assert torch.allclose(vc.float().cpu(), vexp.to(dtype).float(), atol=0, rtol=0)
    # q only (another entry's cache is read): nothing is written
    q2 = torch.empty((T, Hq * hd), dtype=dtype, device=dev())
    ops.rope_kv_write(qkv[:, : Hq * hd].contiguous(), pos, None, inv, rd, inter, q2, None, None, Hq, Hkv, hd)
    assert torch.equal(q2, q)


def paged_setup(dtype, lens, starts, Hq, Hkv, hd, page, seed, spike=False):
    """Random requests laid out in shuffled pages.  Returns what the kernel needs and, per
    request, the contiguous q, k, v of its whole context for the plain reference."""
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    ctx = [s + n for s, n in zip(starts, lens)]
    max_pages = max(-(-c // page) for c in ctx) + 1
    total_pages = sum(-(-c // page) for c in ctx) + 3
    perm = torch.randperm(total_pages, generator=g).tolist()
    kc = torch.full((total_pages * page, Hkv, hd), float("nan"), dtype=torch.float32)
    vc = torch.full((total_pages * page, Hkv, hd), float("nan"), dtype=torch.float32)
    bt = torch.full((S, max_pages), -1, dtype=torch.int32)
    full = []
    rows = 0
    for i in range(S):
        k = torch.randn((ctx[i], Hkv, hd), generator=g).to(dtype).float()
        v = torch.randn((ctx[i], Hkv, hd), generator=g).to(dtype).float()
        qf = torch.randn((ctx[i], Hq, hd), generator=g).to(dtype).float()
        if spike:  # one far key stands out for the last query: a stale or skipped page shows
            far = min(3, ctx[i] - 1)
            k[far] = 0
            k[far, :, 0] = 8.0
            qf[-1] = 0
            qf[-1, :, 0] = 8.0
            v[far] = 5.0
        for lp in range(-(-ctx[i] // page)):
            phys = perm.pop()
            bt[i, lp] = phys
            n = min(page, ctx[i] - lp * page)
            kc[phys * page: phys * page + n] = k[lp * page: lp * page + n]
            vc[phys * page: phys * page + n] = v[lp * page: lp * page + n]
        full.append((qf, k, v))
        rows += lens[i]
    q = torch.cat([full[i][0][starts[i]:] for i in range(S)], dim=0)
    d = dev()
    span_row = torch.tensor(np.cumsum([0] + lens[:-1]), dtype=torch.int32, device=d)
    return dict(q=q.to(dtype).to(d).reshape(rows, Hq * hd), kc=kc.to(dtype).to(d), vc=vc.to(dtype).to(d),
                bt=bt.to(d), max_pages=max_pages, span_row=span_row,
                span_len=torch.tensor(lens, dtype=torch.int32, device=d),
                span_pos=torch.tensor(starts, dtype=torch.int32, device=d), full=full, rows=rows)


def attention_reference(full, lens, starts, hd, window):
    outs = []
    for (qf, k, v), n, s in zip(full, lens, starts):
        o = plain_attention(qf, k, v, 1.0 / math.sqrt(hd), window)
        outs.append(o[s:])
    return torch.cat(outs, dim=0)


def tiles_for(lens, bq):
    ts, tq = [], []
    for i, n in enumerate(lens):
        for q0 in range(0, n, bq):
            ts.append(i)
            tq.append(q0)
    d = dev()
    return torch.tensor(ts, dtype=torch.int32, device=d), torch.tensor(tq, dtype=torch.int32, device=d), len(ts)


ATTN_CASES = [
    # Hq, Hkv, hd, page, lens, starts, window, bq
    (4, 2, 16, 16, [5, 17, 33], [0, 0, 0], None, 8),
    (3, 1, 32, 8, [1, 9, 40, 2], [70, 0, 31, 64], None, 4),
    (14, 2, 64, 16, [1, 1, 50], [300, 15, 200], None, 16),
    (5, 5, 48, 16, [1, 30, 3], [100, 17, 19], 20, 8),
    (6, 3, 80, 4, [2, 64], [62, 0], 7, 2),
    (8, 1, 128, 16, [7, 1], [9, 500], None, 4),
    # one query row per tile: the decode kernel
    (14, 2, 64, 16, [1, 1, 1], [300, 15, 0], None, 1),
    (3, 1, 32, 8, [1, 1], [70, 5], None, 1),
    (5, 5, 48, 16, [1, 1, 1], [100, 17, 19], 20, 1),
    (16, 1, 128, 16, [1, 1], [130, 31], None, 1),
    (8, 2, 256, 32, [1], [200], 64, 1),
    (6, 3, 20, 4, [1, 1], [62, 3], None, 1),          # head size the 16-byte loads refuse: general kernel
]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("case", ATTN_CASES)
@pytest.mark.parametrize("spike", [False, True])
def test_paged_attention_simt(ops, dtype, case, spike):
    Hq, Hkv, hd, page, lens, starts, window, bq = case
    s = paged_setup(dtype, lens, starts, Hq, Hkv, hd, page, seed=21, spike=spike)
    ts, tq, nt = tiles_for(lens, bq)
    out = torch.full((s["rows"], Hq * hd), float("nan"), dtype=dtype, device=dev())
    ops.paged_attention_simt(s["q"], s["kc"], s["vc"], out, ts, tq, nt, s["span_row"], s["span_len"], s["span_pos"],
                             s["bt"], s["max_pages"], page, Hq, Hkv, hd, window or 0, 1.0 / math.sqrt(hd), bq)
    ref = attention_reference(s["full"], lens, starts, hd, window).reshape(s["rows"], Hq * hd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    got = out.float().cpu()
    assert not torch.isnan(got).any()
    assert torch.allclose(got, ref, atol=tol, rtol=tol), f"max diff {float((got - ref).abs().max())}"


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("nsplit", [2, 5, 16])
@pytest.mark.parametrize("window", [None, 100])
def test_paged_attention_split(ops, dtype, nsplit, window):
    Hq, Hkv, hd, page = 14, 2, 64, 16
    lens, starts = [1, 1, 1, 1], [700, 0, 33, 257]
    s = paged_setup(dtype, lens, starts, Hq, Hkv, hd, page, seed=22, spike=True)
    ts, tq, nt = tiles_for(lens, 1)
    out = torch.full((4, Hq * hd), float("nan"), dtype=dtype, device=dev())
    scratch = torch.empty(ops.attention_scratch_floats(nt, Hq, hd, 1, nsplit), dtype=torch.float32, device=dev())
    ops.paged_attention_simt(s["q"], s["kc"], s["vc"], out, ts, tq, nt, s["span_row"], s["span_len"], s["span_pos"],
                             s["bt"], s["max_pages"], page, Hq, Hkv, hd, window or 0, 1.0 / math.sqrt(hd), 1,
                             nsplit, scratch)
    ref = attention_reference(s["full"], lens, starts, hd, window).reshape(4, Hq * hd)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    got = out.float().cpu()
    assert torch.allclose(got, ref, atol=tol, rtol=tol), f"max diff {float((got - ref).abs().max())}"


TC_ATTN_CASES = [
    # Hq, Hkv, hd, page, lens, starts, window
    (2, 1, 64, 16, [128], [0], None),
    (14, 2, 64, 16, [300, 40, 129], [0, 77, 500], None),
    (4, 4, 64, 8, [33, 250], [1000, 3], 100),
    (6, 2, 128, 32, [200, 64], [5, 130], None),
    (3, 1, 128, 16, [512], [0], 130),
    (2, 2, 64, 128, [260], [40], None),
]


@pytest.mark.parametrize("case", TC_ATTN_CASES)
@pytest.mark.parametrize("spike", [False, True])
def test_paged_attention_tcgen05(ops, case, spike):
    Hq, Hkv, hd, page, lens, starts, window = case
    assert ops.attention_tcgen05_supports(hd, page)
    s = paged_setup(torch.bfloat16, lens, starts, Hq, Hkv, hd, page, seed=23, spike=spike)
    ts, tq, nt = tiles_for(lens, 128)
    out = torch.full((s["rows"], Hq * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    ops.paged_attention_tcgen05(s["q"], s["kc"], s["vc"], out, ts, tq, nt, s["span_row"], s["span_len"], s["span_pos"],
                                s["bt"], s["max_pages"], page, Hq, Hkv, hd, window or 0, 1.0 / math.sqrt(hd))
    ops.check_async_errors(dev())
    ref = attention_reference(s["full"], lens, starts, hd, window).reshape(s["rows"], Hq * hd)
    got = out.float().cpu()
    assert not torch.isnan(got).any()
    assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), f"max diff {float((got - ref).abs().max())}"


@pytest.mark.parametrize("window", [None, 300])
@pytest.mark.parametrize("chunk_tiles", [1, 2, 4])
def test_paged_attention_tcgen05_cut_key_ranges(ops, window, chunk_tiles):
    """Long key ranges cut into work items whose partial results a second kernel merges."""
    from lightllm_b200.engine.batch import Span, StepContext
    Hq, Hkv, hd, page = 6, 2, 64, 16
    lens, starts = [1100, 40, 700], [0, 900, 333]
    s = paged_setup(torch.bfloat16, lens, starts, Hq, Hkv, hd, page, seed=27, spike=True)
    ctx = StepContext()
    ctx.device = dev()
    rows = 0
    for i, (n, st) in enumerate(zip(lens, starts)):
        ctx.spans.append(Span(i, i, st, n, rows))
        rows += n
    ctx.iota = torch.arange(3, dtype=torch.int32, device=dev())
    ctx.zeros = torch.zeros(3, dtype=torch.int32, device=dev())
    ts, tq, nt, cut = ctx.attention_items(32, window or 0, chunk_tiles)
    if window is None or chunk_tiles < 3:
        assert cut is not None and cut[3] > 0 and nt > len(tiles_for(lens, 128)[0])
    out = torch.full((s["rows"], Hq * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    ops.paged_attention_tcgen05(s["q"], s["kc"], s["vc"], out, ts, tq, nt, s["span_row"], s["span_len"], s["span_pos"],
                                s["bt"], s["max_pages"], page, Hq, Hkv, hd, window or 0, 1.0 / math.sqrt(hd), cut=cut)
    ops.check_async_errors(dev())
    ref = attention_reference(s["full"], lens, starts, hd, window).reshape(s["rows"], Hq * hd)
    got = out.float().cpu()
    assert not torch.isnan(got).any()
    assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), f"max diff {float((got - ref).abs().max())}"


def test_attention_tcgen05_refuses_other_shapes(ops):
    assert not ops.attention_tcgen05_supports(48, 16) and not ops.attention_tcgen05_supports(64, 24)
    z = torch.zeros((4, 48), dtype=torch.bfloat16, device=dev())
    i = torch.zeros(1, dtype=torch.int32, device=dev())
    with pytest.raises(ops.KernelError, match="not supported"):
        ops.paged_attention_tcgen05(z, z.view(4, 1, 48), z.view(4, 1, 48), z, i, i, 1, i, i, i, i.view(1, 1), 1, 16,
                                    1, 1, 48, 0, 1.0)


MMA_DECODE_CASES = [
    # Hq, Hkv, hd, page, starts (context = start + 1), window
    (14, 2, 64, 16, [300, 15, 0, 2047], None),
    (12, 2, 128, 16, [700, 31, 32], None),
    (28, 4, 128, 8, [100, 1], 64),
    (16, 1, 64, 32, [513, 64, 5], None),
    (4, 4, 64, 16, [129], 100),
    (3, 1, 64, 4, [77, 78, 79, 80, 81], None),
]


@pytest.mark.parametrize("case", MMA_DECODE_CASES)
@pytest.mark.parametrize("nsplit", [1, 3, 8, 16, 20])      # up to 16 merged inside the kernel, beyond by the merge kernel
@pytest.mark.parametrize("spike", [False, True])
def test_paged_decode_mma(ops, case, nsplit, spike):
    Hq, Hkv, hd, page, starts, window = case
    assert ops.paged_decode_mma_supports(Hq, Hkv, hd)
    lens = [1] * len(starts)
    s = paged_setup(torch.bfloat16, lens, starts, Hq, Hkv, hd, page, seed=25, spike=spike)
    ts, tq, nt = tiles_for(lens, 1)
    out = torch.full((s["rows"], Hq * hd), float("nan"), dtype=torch.bfloat16, device=dev())
    scratch = None
    if nsplit > ops.decode_mma_cluster_splits():
        scratch = torch.empty(ops.attention_scratch_floats(nt, Hq, hd, 1, nsplit), dtype=torch.float32, device=dev())
    ops.paged_decode_mma(s["q"], s["kc"], s["vc"], out, ts, tq, nt, s["span_row"], s["span_pos"], s["bt"],
                         s["max_pages"], page, Hq, Hkv, hd, window or 0, 1.0 / math.sqrt(hd), nsplit, scratch)
    ref = attention_reference(s["full"], lens, starts, hd, window).reshape(s["rows"], Hq * hd)
    got = out.float().cpu()
    assert not torch.isnan(got).any()
    assert torch.allclose(got, ref, atol=2e-2, rtol=2e-2), f"max diff {float((got - ref).abs().max())}"


@pytest.mark.parametrize("V", [151937, 16384, 1003])      # long rows are shared among blocks, short ones are not
def test_argmax_lowest_index_on_ties(ops, V):
    x = rnd((9, V), torch.float32, 30)
    x[0, 100] = x[0, 900] = 50.0
    x[1, V - 1] = 60.0
    x[2, :] = 1.0
    x[3, :] = float("-inf")                      # nothing above -inf: index 0
    x[4, :] = -3.0
    x[4, V // 2] = -0.0                          # the zeros are equal: the first of them
    x[4, V - 7] = 0.0
    x[5, :] = float("-inf")
    x[5, V - 2] = -1e30
    x[6, V // 3] = float("nan")                  # a NaN is never the largest
    if V > 4096:
        x[7, 4095] = x[7, 4096] = 70.0           # a tie across two blocks' pieces
    out = torch.full((9,), -1, dtype=torch.int32, device=dev())
    for _ in range(2):                           # the second run finds the meeting place clean
        ops.argmax(x, out)
        got = out.cpu().tolist()
        ref = [int(np.argmax(np.nan_to_num(r, nan=-np.inf))) for r in x.cpu().numpy()]
        assert got == ref
        assert got[0] == 100 and got[2] == 0 and got[3] == 0 and got[4] == V // 2 and got[5] == V - 2
        out.fill_(-1)
    scratch = ops._argmax_scratch.get(dev().index or 0)
    assert scratch is None or int(scratch.abs().max()) == 0


@pytest.mark.parametrize("temperature,top_k,top_p,min_p", [(1.0, 0, 1.0, 0.0), (0.7, 40, 1.0, 0.0),
                                                           (1.3, 0, 0.9, 0.0), (1.0, 0, 1.0, 0.05),
                                                           (0.8, 50, 0.95, 0.02), (0.0, 0, 1.0, 0.0)])
@pytest.mark.parametrize("V", [1003, 20011, 151936])      # one block per row; from 8,192 on a cluster of blocks per row
def test_sample_matches_plain_distribution(ops, temperature, top_k, top_p, min_p, V):
    """For many uniform numbers the kernel picks the token that the plain inverse-CDF draw picks
    from the plain filtered distribution (up to draws that fall within rounding of a boundary)."""
    R = 256
    g = torch.Generator().manual_seed(31)
    logits_row = torch.randn(V, generator=g) * 3.0
    logits = logits_row[None, :].repeat(R, 1).contiguous().to(dev())
    u = (torch.arange(R, dtype=torch.float32) + 0.5) / R
    out = torch.empty(R, dtype=torch.int32, device=dev())
    f = lambda v: torch.full((R,), v, dtype=torch.float32, device=dev())
    ops.sample(logits, f(temperature), torch.full((R,), top_k, dtype=torch.int32, device=dev()), f(top_p), f(min_p),
               u.to(dev()), out)
    got = out.cpu().tolist()
    if temperature < 1e-5:
        assert set(got) == {int(torch.argmax(logits_row))}
        return
    p = plain_sampling_probs(logits_row.numpy(), temperature, top_k, top_p, min_p)
    ref = [plain_draw(p, float(x)) for x in u]
    cdf = np.cumsum(p)
    wrong = 0
    for gi, ri, x in zip(got, ref, u.tolist()):
        assert p[gi] > 0.0, "a filtered token was drawn"
        if gi != ri:
            near = min(abs(cdf[min(gi, ri)] - x), abs(cdf[max(gi, ri) - 1] - x) if max(gi, ri) > 0 else 1.0)
            assert near < 1e-4, f"u={x}: kernel {gi}, plain {ri}"
            wrong += 1
    # a long row has its boundaries closer together (thousands of tokens share the mass), so more of the 256 draws
    # fall within float rounding of one
    assert wrong <= (3 if V < 8192 else 16)


def test_sample_rows_have_their_own_parameters(ops):
    """Rows of one launch with different temperatures, filters and uniform numbers (greedy rows among them), over a
    long row: each row is drawn as the plain implementation draws it."""
    V = 30011
    rows = [(0.7, 0, 1.0, 0.0, 0.31), (0.0, 0, 1.0, 0.0, 0.5), (1.2, 25, 1.0, 0.0, 0.77), (0.9, 0, 0.8, 0.0, 0.05),
            (1.0, 0, 1.0, 0.1, 0.93), (0.8, 300, 0.9, 0.01, 0.61), (1.5, 1, 1.0, 0.0, 0.99), (1.0, 0, 1.0, 0.0, 0.999999)]
    g = torch.Generator().manual_seed(77)
    logits = (torch.randn(len(rows), V, generator=g) * 2.5).contiguous()
    col = lambda j, dt: torch.tensor([r[j] for r in rows], dtype=dt, device=dev())
    out = torch.empty(len(rows), dtype=torch.int32, device=dev())
    ops.sample(logits.to(dev()), col(0, torch.float32), col(1, torch.int32), col(2, torch.float32), col(3, torch.float32),
               col(4, torch.float32), out)
    for i, (t, k, tp, mp, u) in enumerate(rows):
        got = int(out[i])
        if t < 1e-5:
            assert got == int(torch.argmax(logits[i]))
            continue
        p = plain_sampling_probs(logits[i].numpy(), t, k, tp, mp)
        ref = plain_draw(p, u)
        assert p[got] > 0.0, f"row {i}: a filtered token was drawn"
        if got != ref:
            cdf = np.cumsum(p)
            near = min(abs(cdf[min(got, ref)] - u), abs(cdf[max(got, ref) - 1] - u))
            assert near < 1e-4, f"row {i}: kernel {got}, plain {ref}"


def test_a_wait_that_runs_out_is_reported_and_the_library_goes_on(ops):
    """The block of csrc/selftest.cu waits on a barrier that nothing completes, with a limit of a million cycles: one
    role's limit runs out, the other leaves because the first gave up, tensor memory is freed, the host reads the
    flag; the next ordinary kernels (a tensor-core contraction among them) run and the flag stays clear."""
    ops.check_async_errors(dev())                       # clear before the test
    trace = ops.selftest_wait_expires(dev(), 1_000_000)
    with pytest.raises(ops.KernelError, match="gave up waiting"):
        ops.check_async_errors(dev())
    assert trace.cpu().tolist() == [2, 2]
    ops.check_async_errors(dev())                       # the flag was cleared by the report
    a, w = rnd((8, 128), torch.bfloat16, 41), rnd((256, 128), torch.bfloat16, 42)
    out = torch.empty((8, 256), dtype=torch.float32, device=dev())
    ops.gemm_decode(w, ops.DEPI_STORE_F32, 8, a=a, out=out)
    ops.check_async_errors(dev())
    ref = a.float().cpu() @ w.float().cpu().t()
    assert torch.allclose(out.cpu(), ref, atol=2e-2, rtol=2e-2)


# ---------------------------------------------------------------------------------------------
# The layers of a decode step as one persistent kernel
# ---------------------------------------------------------------------------------------------
FUSED_CASES = [
    # D, Hq, Hkv, hd, I, page, rotary_dim, interleaved, bias, norm dtype, window, layers, contexts (keys before the new token)
    (136, 6, 2, 64, 344, 16, 64, False, True, torch.bfloat16, None, 2, [0, 1, 15, 16, 17, 300, 700]),
    (256, 4, 2, 128, 520, 8, 128, False, True, torch.bfloat16, 150, 2, [5, 149, 150, 151, 400]),
    (192, 3, 1, 64, 136, 32, 32, True, False, torch.float32, None, 3, [0, 2100]),
    (128, 16, 1, 64, 256, 16, 64, False, True, torch.bfloat16, None, 1, list(range(0, 64 * 9, 9))),        # 64 rows
    (128, 2, 2, 128, 64, 16, 0, False, False, torch.bfloat16, 40, 2, [33 * i for i in range(20)]),          # 20 rows, no positions
    # wide layers: a block owns more tiles of a stage than its ring holds and parts of several row tiles, so operands
    # are built in several batches and accumulators are drained while later ones are still being fed
    (2048, 16, 2, 128, 8192, 16, 128, False, True, torch.bfloat16, None, 1, [5, 300, 17]),
    (1024, 8, 8, 64, 4096, 16, 64, False, True, torch.bfloat16, None, 2, [40 + 3 * i for i in range(40)]),  # the same at 40 rows
]


def fused_reference(h, layers, ctx_k, ctx_v, positions, Hq, Hkv, hd, rotary_dim, interleaved, theta, window):
    """Plain float64 layers on the new tokens: h [M, D]; ctx_k/ctx_v[l][r]: the cached keys and values of request r."""
    from tests.plain import qwen2_plain as P
    M = h.shape[0]
    new_k = [[None] * M for _ in layers]
    new_v = [[None] * M for _ in layers]
    for li, w in enumerate(layers):
        x = P.plain_rmsnorm(h, w["n1"], w["eps1"])
        qkv = P.plain_linear(x, w["w_qkv"], w["b_qkv"])
        q = qkv[:, : Hq * hd].reshape(M, Hq, hd)
        k = qkv[:, Hq * hd: (Hq + Hkv) * hd].reshape(M, Hkv, hd)
        v = qkv[:, (Hq + Hkv) * hd:].reshape(M, Hkv, hd)
        if rotary_dim:
            q = P.plain_rope(q, positions, theta, rotary_dim, interleaved=interleaved)
            k = P.plain_rope(k, positions, theta, rotary_dim, interleaved=interleaved)
        att = torch.zeros(M, Hq * hd, dtype=h.dtype)
        for r in range(M):
            kk = torch.cat([ctx_k[li][r], k[r: r + 1]])
            vv = torch.cat([ctx_v[li][r], v[r: r + 1]])
            qq = torch.zeros(kk.shape[0], Hq, hd, dtype=h.dtype)
            qq[-1] = q[r]
            att[r] = P.plain_attention(qq, kk, vv, 1.0 / math.sqrt(hd), window)[-1].reshape(-1)
            new_k[li][r], new_v[li][r] = k[r], v[r]
        h = h + P.plain_linear(att, w["w_o"])
        x = P.plain_rmsnorm(h, w["n2"], w["eps2"])
        h = h + P.plain_swiglu(x, w["w_gate"], w["w_up"], w["w_down"])
    return h, new_k, new_v


@pytest.mark.parametrize("case", FUSED_CASES)
def test_decode_layers_against_plain_layers(ops, case):
    """The persistent kernel on its own, at sizes the engine's tests do not have: first tokens, page edges, a window's
    edge, 64 rows, groups of 16, partial and interleaved rotation, float32 norm weights, no bias, no positions.  The
    residual after the layers and the keys and values it wrote are compared with plain float64 layers.  Run twice:
    the second launch finds the scratch and the counters as the first left them."""
    D, Hq, Hkv, hd, I, page, rotary_dim, interleaved, bias, norm_dt, window, nl, contexts = case
    M = len(contexts)
    assert ops.decode_layers_supports(M, D, Hq, Hkv, hd, I, rotary_dim)
    g = torch.Generator().manual_seed(50 + D)
    bf = lambda t: t.to(torch.bfloat16)
    rn = lambda *shape, s=1.0: torch.randn(*shape, generator=g) * s
    theta = 10000.0
    Nqkv = (Hq + 2 * Hkv) * hd
    total_pages = sum(-(-(c + 1) // page) for c in contexts) + 2
    perm = torch.randperm(total_pages, generator=g).tolist()
    max_pages = max(-(-(c + 1) // page) for c in contexts) + 1
    bt = torch.full((M, max_pages), -1, dtype=torch.int32)
    for r, c in enumerate(contexts):
        for lp in range(-(-(c + 1) // page)):
            bt[r, lp] = perm.pop()
    slot = torch.tensor([int(bt[r, c // page]) * page + c % page for r, c in enumerate(contexts)], dtype=torch.int32)
    layers, ref_layers, caches, ctx_k, ctx_v = [], [], [], [], []
    for li in range(nl):
        w = dict(w_qkv=bf(rn(Nqkv, D, s=D ** -0.5)), w_o=bf(rn(D, Hq * hd, s=(Hq * hd) ** -0.5)),
                 w_gate=bf(rn(I, D, s=D ** -0.5)), w_up=bf(rn(I, D, s=D ** -0.5)), w_down=bf(rn(D, I, s=I ** -0.5)),
                 b_qkv=rn(Nqkv, s=0.3) if bias else None, n1=(1 + rn(D, s=0.1)).to(norm_dt), n2=(1 + rn(D, s=0.1)).to(norm_dt),
                 eps1=1e-5, eps2=3e-6)
        kc = torch.full((total_pages * page, Hkv, hd), float("nan"))       # rows that no request owns stay NaN
        vc = torch.full((total_pages * page, Hkv, hd), float("nan"))
        ks, vs = [], []
        for r, c in enumerate(contexts):
            k, v = bf(rn(c, Hkv, hd)).float(), bf(rn(c, Hkv, hd)).float()
            if c > 3:           # a far key that matters: a piece that is lost or weighted wrongly shows
                k[2] = 0.0
                k[2, :, 0] = 6.0
                v[2] = 4.0
            for pos in range(c):
                at = int(bt[r, pos // page]) * page + pos % page
                kc[at], vc[at] = k[pos], v[pos]
            ks.append(k.double())
            vs.append(v.double())
        ctx_k.append(ks)
        ctx_v.append(vs)
        kc, vc = bf(kc).to(dev()), bf(vc).to(dev())
        caches.append((kc, vc))
        dw = {k: (v.to(dev()) if isinstance(v, torch.Tensor) else v) for k, v in w.items()}
        layers.append(dict(w_qkv=dw["w_qkv"], w_o=dw["w_o"],
                           w_gate_up=torch.stack([dw["w_gate"], dw["w_up"]], dim=1).reshape(2 * I, D).contiguous(),
                           w_down=dw["w_down"], b_qkv=dw["b_qkv"], norm1_w=dw["n1"], norm2_w=dw["n2"], k_cache=kc, v_cache=vc,
                           eps1=w["eps1"], eps2=w["eps2"], window=window or 0, group=0))
        ref_layers.append({k: (v.double() if isinstance(v, torch.Tensor) else v) for k, v in w.items()})
    h0 = rn(M, D, s=2.0)
    positions = torch.tensor(contexts, dtype=torch.int32)
    want, new_k, new_v = fused_reference(h0.double(), ref_layers, ctx_k, ctx_v, positions.long(), Hq, Hkv, hd, rotary_dim,
                                         interleaved, theta, window)
    desc = ops.decode_layers_descriptors(layers, D, Hq, Hkv, hd, I, dev())
    counters = ops.decode_layers_counters(dev())
    nsplit = 5 if max(contexts) > 256 else 2
    scratch = torch.full((ops.decode_layers_scratch_floats(M, Hq, Hkv, hd, I, nsplit),), float("nan"), device=dev())
    table = None
    if rotary_dim:
        inv_freq = (1.0 / theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float64) / rotary_dim)).float().to(dev())
        table = ops.rope_table(positions.to(dev()), inv_freq)
    for attempt in range(2):
        h = h0.clone().to(dev())
        ops.decode_layers(desc, nl, h, D, Hq, Hkv, hd, I, rotary_dim, interleaved, 1.0 / math.sqrt(hd), table,
                          positions.to(dev()), [bt.to(dev())], [slot.to(dev())], max_pages, page, nsplit, scratch, counters)
        ops.check_async_errors(dev())
        assert counters.cpu().tolist() == [0, 0]
        got = h.cpu().double()
        assert not torch.isnan(got).any()
        scale = float(want.abs().max())
        err = float((got - want).abs().max())
        assert err <= 3e-2 * scale, f"attempt {attempt}: residual differs by {err} (largest value {scale})"
        for li, (kc, vc) in enumerate(caches):
            for r in range(M):
                at = int(slot[r])
                assert torch.allclose(kc[at].cpu().double(), new_k[li][r], atol=3e-2, rtol=3e-2), (li, r)
                assert torch.allclose(vc[at].cpu().double(), new_v[li][r], atol=3e-2, rtol=3e-2), (li, r)


def test_decode_layers_refuses_what_it_cannot_run(ops):
    assert not ops.decode_layers_supports(65, 128, 2, 2, 64, 64, 64)          # too many rows
    assert not ops.decode_layers_supports(4, 128, 2, 2, 48, 64, 48)           # a head size without a kernel
    assert not ops.decode_layers_supports(4, 132, 2, 2, 64, 64, 64)           # a width whose rows are not 16-byte multiples
    assert not ops.decode_layers_supports(4, 128, 34, 2, 64, 64, 64)          # groups of 17
    h = torch.zeros((4, 128), dtype=torch.float32, device=dev())
    i32 = torch.zeros((4, 1), dtype=torch.int32, device=dev())
    with pytest.raises(ops.KernelError, match="unsupported sizes"):
        ops.decode_layers(torch.zeros(1024, dtype=torch.uint8, device=dev()), 1, h, 128, 2, 2, 48, 64, 48, False, 1.0, None,
                          i32.view(-1), [i32], [i32.view(-1)], 1, 16, 1, torch.zeros(8, device=dev()),
                          ops.decode_layers_counters(dev()))


@pytest.mark.parametrize("n,a_tmem,neighbours,kind", [(64, False, 0, 1), (128, False, 8, 2), (64, True, 4, 1), (16, False, 8, 1)])
def test_mma_issue_microbenchmark(ops, n, a_tmem, neighbours, kind):
    """The issue-cost microbenchmark runs, ends by itself and reports plausible cycle counts (an MMA of this shape
    keeps the tensor pipe for 32-64 cycles; beside busy warps the issuing thread needs a multiple)."""
    r = ops.selftest_mma_issue(dev(), n, a_tmem, neighbours, kind, iters=64)
    torch.cuda.synchronize()
    ops.check_async_errors(dev())
    assert 20.0 < r["cycles_per_mma"] < 5000.0 and 0 < r["commit_cycles"] < 100000

