"""``bench_ops [--rows T] [--batch B] [--context C] [--reps N] [--only NAME ...]``: every kernel of the library alone.

The reference times its operators one by one in its test program (tests/test_ops.cu:92-231: add, SiLU, RMSNorm,
rotation, contractions).  This tool does the same for this library's kernels at the layer sizes of a configuration
(by default the Qwen2.5-0.5B sizes): each operator runs ``--reps`` times between CUDA events, after a warm-up, with a
buffer larger than L2 written in between so that every run starts cold, and is reported with the bytes it has to move
and the bandwidth that makes.  It is also the workload under which the kernels' profiler summaries are taken (one
operator with ``--only``).
"""
import argparse
import json
import math
import sys

SIZES = {"hidden": 896, "heads": 14, "kv_heads": 2, "head_dim": 64, "intermediate": 4864, "vocab": 151936, "page": 16}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bench_ops")
    ap.add_argument("--rows", type=int, default=2048, help="rows of a prompt portion (prefill-shaped operators)")
    ap.add_argument("--batch", type=int, default=8, help="requests of a decode step (decode-shaped operators)")
    ap.add_argument("--context", type=int, default=2048, help="keys each request holds (attention operators)")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--only", nargs="*", default=None, help="names of the operators to run (default: all)")
    for k, v in SIZES.items():
        ap.add_argument(f"--{k.replace('_', '-')}", type=int, default=v)
    args = ap.parse_args(argv)

    import torch
    from lightllm_b200.csrc import ops
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    rn = lambda *shape, dtype=torch.float32, s=1.0: (torch.randn(*shape, generator=g, device=dev) * s).to(dtype)
    T, B, C = args.rows, args.batch, args.context
    D, Hq, Hkv, hd, I, V, page = (args.hidden, args.heads, args.kv_heads, args.head_dim, args.intermediate, args.vocab,
                                  args.page)
    Nqkv = (Hq + 2 * Hkv) * hd
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=dev)          # larger than L2
    results = []

    def run(name, fn, nbytes, flops=0):
        if args.only and name not in args.only:
            return
        for _ in range(3):
            fn()
        times = []
        for _ in range(args.reps):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1) * 1000.0)
        times.sort()
        us = times[len(times) // 2]
        rec = {"op": name, "us": round(us, 2), "MB": round(nbytes / 1e6, 3), "GB/s": round(nbytes / us / 1e3, 1)}
        if flops:
            rec["TFLOP/s"] = round(flops / us / 1e6, 2)
        results.append(rec)
        print(json.dumps(rec), flush=True)

    # ---- what a prompt portion of T rows runs ---------------------------------------------------------------------------
    ids = torch.randint(0, V, (T,), generator=g, device=dev, dtype=torch.int32)
    table = rn(V, D, dtype=torch.bfloat16, s=0.02)
    resid = torch.empty((T, D), dtype=torch.float32, device=dev)
    run("embedding", lambda: ops.embedding(ids, table, resid), T * D * (2 + 4))
    w_norm = torch.ones(D, dtype=torch.bfloat16, device=dev)
    x_bf = torch.empty((T, D), dtype=torch.bfloat16, device=dev)
    run("rmsnorm", lambda: ops.rmsnorm(resid, w_norm, 1e-6, x_bf), T * D * (4 + 2))
    resid32 = rn(T, D)
    w_norm32 = torch.ones(D, device=dev)
    x32 = torch.empty((T, D), device=dev)
    run("rmsnorm_float32", lambda: ops.rmsnorm(resid32, w_norm32, 1e-6, x32), T * D * 8)
    positions = torch.arange(T, dtype=torch.int32, device=dev)
    inv_freq = (1.0 / 1e6 ** (torch.arange(0, hd, 2, dtype=torch.float64) / hd)).float().to(dev)
    run("rope_table", lambda: ops.rope_table(positions, inv_freq), T * hd // 2 * 8)
    slots = -(-T // page) * page
    kc = torch.zeros((slots, Hkv, hd), dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    qkv = rn(T, Nqkv, dtype=torch.bfloat16)
    q_out = torch.empty((T, Hq * hd), dtype=torch.bfloat16, device=dev)
    run("rope_kv_write", lambda: ops.rope_kv_write(qkv, positions, positions, inv_freq, hd, False, q_out, kc, vc, Hq, Hkv, hd),
        2 * T * Nqkv * 2)
    # the 32-bit contraction and attention (the float32 path), at a portion of 256 rows so that a run stays short
    Ts = min(T, 256)
    a32, w32 = rn(Ts, D), rn(Nqkv, D, s=D ** -0.5)
    out32 = torch.empty((Ts, Nqkv), device=dev)
    run("gemm_simt_float32", lambda: ops.gemm_simt(a32, w32, None, ops.EPI_STORE, out32), (Ts * D + Nqkv * D + Ts * Nqkv) * 4,
        2 * Ts * D * Nqkv)
    kc32, vc32 = rn(slots, Hkv, hd), rn(slots, Hkv, hd)
    q32, o32 = rn(Ts, Hq * hd), torch.empty((Ts, Hq * hd), device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
    bt = torch.arange(slots // page, dtype=torch.int32, device=dev).reshape(1, -1)
    bq = 16
    tiles = list(range(0, Ts, bq))
    run("paged_attention_simt_float32",
        lambda: ops.paged_attention_simt(q32, kc32, vc32, o32, i32([0] * len(tiles)), i32(tiles), len(tiles), i32([0]), i32([Ts]),
                                         i32([0]), bt, bt.shape[1], page, Hq, Hkv, hd, 0, 1 / math.sqrt(hd), bq),
        (2 * Ts * Hq * hd + 2 * Ts * Hkv * hd) * 4, 2 * 2 * Hq * hd * Ts * (Ts + 1) // 2)

    # the four contractions of a layer on the tensor cores, as a portion of T rows runs them (K cut as the engine cuts it)
    if ops.has_tcgen05() and T > 128:
        from lightllm_b200.parts import linear as L
        resid_f = rn(T, D)
        w_qkv, b_qkv = rn(Nqkv, D, dtype=torch.bfloat16, s=D ** -0.5), rn(Nqkv)
        w_o = rn(D, Hq * hd, dtype=torch.bfloat16, s=(Hq * hd) ** -0.5)
        w_gu = rn(2 * I, D, dtype=torch.bfloat16, s=D ** -0.5)
        w_dn = rn(D, I, dtype=torch.bfloat16, s=I ** -0.5)
        x_in, attn_o = rn(T, D, dtype=torch.bfloat16), rn(T, Hq * hd, dtype=torch.bfloat16)
        act = torch.empty((T, I), dtype=torch.bfloat16, device=dev)
        qkv_out = torch.empty((T, Nqkv), dtype=torch.bfloat16, device=dev)
        gemm_bytes = lambda M, N, K, out_b: (M * K + N * K) * 2 + M * N * out_b
        run("gemm_tcgen05_qkv", lambda: L.linear(x_in, w_qkv, b_qkv, L.STORE, qkv_out), gemm_bytes(T, Nqkv, D, 2), 2 * T * Nqkv * D)
        run("gemm_tcgen05_o_proj_residual", lambda: L.linear(attn_o, w_o, None, L.RESIDUAL, residual=resid_f),
            gemm_bytes(T, D, Hq * hd, 8), 2 * T * D * Hq * hd)
        run("gemm_tcgen05_gate_up_swiglu", lambda: L.linear(x_in, w_gu, None, L.SWIGLU, act), gemm_bytes(T, 2 * I, D, 1),
            2 * T * 2 * I * D)
        run("gemm_tcgen05_down_residual", lambda: L.linear(act, w_dn, None, L.RESIDUAL, residual=resid_f), gemm_bytes(T, D, I, 8),
            2 * T * D * I)
        for sk in (1, 2, 4):
            run(f"gemm_tcgen05_down_residual_split{sk}", lambda: ops.gemm_tcgen05(act, w_dn, None, ops.EPI_RESIDUAL, None, resid_f, sk),
                gemm_bytes(T, D, I, 8), 2 * T * D * I)

    # the tensor-core attention of the whole portion (a prompt of T rows from position 0), cut into items as the engine does
    if ops.attention_tcgen05_supports(hd, page):
        from lightllm_b200.engine.batch import cut_attention_rows
        from lightllm_b200.parts import linear as L
        import numpy as np
        rows_t = [(0, q0, -(-min(q0 + 128, T) // 128)) for q0 in range(0, T, 128)]
        items, merges, parts = cut_attention_rows(rows_t, None, Hq, (2 if hd <= 64 else 1) * L.num_sms(dev))
        arr = torch.from_numpy(np.asarray([t[1:] for t in items], dtype=np.int32).T.copy()).to(dev)
        m = torch.from_numpy(np.asarray(merges, dtype=np.int32).reshape(-1, 4).T.copy()).to(dev)
        cut = (arr[2], arr[3], arr[4], parts, m[0], m[1], m[2], m[3], len(merges)) if merges else (arr[2], arr[3], arr[4], 0, None, None, None, None, 0)
        kcp, vcp = rn(slots, Hkv, hd, dtype=torch.bfloat16), rn(slots, Hkv, hd, dtype=torch.bfloat16)
        qp = rn(T, Hq * hd, dtype=torch.bfloat16)
        op = torch.empty_like(qp)
        btp = torch.arange(slots // page, dtype=torch.int32, device=dev).reshape(1, -1)
        i32p = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
        sr, sl, sp = i32p([0]), i32p([T]), i32p([0])
        run("paged_attention_tcgen05",
            lambda: ops.paged_attention_tcgen05(qp, kcp, vcp, op, arr[0].contiguous(), arr[1].contiguous(), len(items), sr, sl, sp, btp,
                                                btp.shape[1], page, Hq, Hkv, hd, 0, 1 / math.sqrt(hd), cut=cut),
            (2 * T * Hq * hd + 2 * T * Hkv * hd) * 2, 2 * 2 * Hq * hd * T * (T + 1) // 2)

    # ---- what a decode step of B requests over C keys runs --------------------------------------------------------------
    pages_per = -(-(C + 1) // page)
    kcd = rn(B * pages_per * page, Hkv, hd, dtype=torch.bfloat16)
    vcd = rn(B * pages_per * page, Hkv, hd, dtype=torch.bfloat16)
    btd = torch.arange(B * pages_per, dtype=torch.int32, device=dev).reshape(B, pages_per)
    qd = rn(B, Hq * hd, dtype=torch.bfloat16)
    od = torch.empty_like(qd)
    rows, pos, zero = i32(list(range(B))), i32([C] * B), i32([0] * B)
    kv_bytes = B * (C + 1) * Hkv * hd * 2 * 2
    if ops.paged_decode_mma_supports(Hq, Hkv, hd):
        nsplit = max(1, min(8, ops.decode_mma_resident(hd) * 148 // (B * Hkv), -(-(C + 1) // 128)))
        run("paged_decode_mma", lambda: ops.paged_decode_mma(qd, kcd, vcd, od, rows, zero, B, rows, pos, btd, pages_per, page, Hq,
                                                             Hkv, hd, 0, 1 / math.sqrt(hd), nsplit, None), kv_bytes)
        big = 24           # more pieces than a cluster merges: the pieces meet in scratch and a second kernel merges them
        scratch = torch.empty(ops.attention_scratch_floats(B, Hq, hd, 1, big), device=dev)
        run("paged_decode_mma_and_merge", lambda: ops.paged_decode_mma(qd, kcd, vcd, od, rows, zero, B, rows, pos, btd, pages_per,
                                                                       page, Hq, Hkv, hd, 0, 1 / math.sqrt(hd), big, scratch),
            kv_bytes + 2 * B * Hq * big * (hd + 2) * 4)
    logits = rn(B, V, s=3.0)
    tok = torch.empty(B, dtype=torch.int32, device=dev)
    run("argmax", lambda: ops.argmax(logits, tok), B * V * 4)
    f = lambda v: torch.full((B,), v, dtype=torch.float32, device=dev)
    temp, top_p, min_p, u = f(0.8), f(0.9), f(0.0), f(0.5)
    top_k = torch.full((B,), 40, dtype=torch.int32, device=dev)
    run("sample_top_k_top_p", lambda: ops.sample(logits, temp, top_k, top_p, min_p, u, tok), B * V * 4)
    run("sample_temperature_only", lambda: ops.sample(logits, temp, None, None, None, u, tok), B * V * 4)
    # ---- what issuing tensor-core instructions costs one thread, alone and beside busy warps (cycles, not bytes) -------
    if not args.only or "mma_issue" in args.only:
        for n, a_tmem in ((64, False), (128, False), (64, True), (16, False)):
            for neighbours, kind in ((0, 1), (4, 2), (8, 2), (4, 1), (8, 1)):
                r = ops.selftest_mma_issue(dev, n, a_tmem, neighbours, kind)
                torch.cuda.synchronize()
                rec = {"op": "mma_issue", "n": n, "a_from": "tmem" if a_tmem else "smem", "busy_warps": neighbours,
                       "busy_kind": ("none" if not neighbours else "fma chains" if kind == 1 else "softmax-like"),
                       "cycles_per_mma": round(r["cycles_per_mma"], 1), "commit_cycles": r["commit_cycles"]}
                print(json.dumps(rec), flush=True)
    ops.check_async_errors(dev)
    return 0


if __name__ == "__main__":
    sys.exit(main())
