"""The step context on the host (no GPU): index arrays staged behind the step's metadata, tiles, and the work items
of the tensor-core attention with their adaptive piece length."""
import numpy as np
import torch

from lightllm_b200.engine.batch import Span, StepContext


def context(spans, staging_words=0):
    ctx = StepContext()
    ctx.device = torch.device("cpu")
    ctx.spans = [Span(i, i, start, length, row) for i, (start, length, row) in enumerate(spans)]
    n = len(spans)
    ctx.iota = torch.arange(n, dtype=torch.int32)
    ctx.zeros = torch.zeros(n, dtype=torch.int32)
    if staging_words:
        host = np.zeros(staging_words + 7, dtype=np.int32)
        dev = torch.from_numpy(host)                 # on the CPU the "copy" is the same memory
        ctx._staging = [host, dev, 7, staging_words + 7]
        ctx._host, ctx._dev = host, dev
    return ctx


def test_staged_arrays_lie_behind_each_other_and_name_their_shapes():
    ctx = context([(0, 5, 0)], staging_words=20)
    a = ctx.stage(np.arange(6, dtype=np.int32).reshape(2, 3))
    b = ctx.stage(np.asarray([9, 8, 7], dtype=np.int32))
    assert a.shape == (2, 3) and a.data_ptr() == ctx._dev.data_ptr() + 7 * 4 and b.data_ptr() == ctx._dev.data_ptr() + 13 * 4
    assert ctx._host[7:16].tolist() == [0, 1, 2, 3, 4, 5, 9, 8, 7] and ctx.staged_words == 9
    assert ctx.shape_key == [(2, 3), (3,)] and not ctx.late_uploads
    big = ctx.stage(np.zeros(30, dtype=np.int32))           # no room left: it goes up on its own
    assert ctx.late_uploads and big.numel() == 30 and ctx._staging[2] == 16
    late = context([(0, 5, 0)])                              # after the copy (no staging): the same
    assert late.stage(np.ones(3, dtype=np.int32)).tolist() == [1, 1, 1] and late.late_uploads


def test_tiles_do_not_cross_spans():
    ctx = context([(0, 5, 0), (10, 1, 5), (3, 40, 6)], staging_words=200)
    ts, tq, n = ctx.tiles(16)
    assert n == 5 and ts.tolist() == [0, 1, 2, 2, 2] and tq.tolist() == [0, 0, 0, 16, 32]
    ts, tq, n = ctx.tiles(16, max_len=5)
    assert n == 2 and ts.tolist() == [0, 1]
    assert ctx.tiles(64)[2] == 3 and ctx.tiles(64)[0] is ctx.iota          # one tile per span: the ready-made arrays
    assert ctx.tiles(16, min_len=100)[2] == 0


def test_attention_items_cover_every_key_tile_once():
    ctx = context([(0, 1000, 0), (700, 40, 1000), (3, 20, 1040)], staging_words=4000)
    for window, chunk in ((0, 1), (0, 2), (0, 4), (300, 2), (0, None)):
        ts, tq, n, cut = ctx.attention_items(32, window, chunk, heads=6, slots=8)
        k0, nk, part, nparts = cut[0], cut[1], cut[2], cut[3]
        seen = {}
        for i in range(n):
            key = (int(ts[i]), int(tq[i]))
            seen.setdefault(key, []).append((int(k0[i]), int(nk[i]), int(part[i])))
        for (span, q0), pieces in seen.items():
            s = ctx.spans[span]
            assert s.length >= 32
            pos0 = s.start + q0
            hi = pos0 + min(128, s.length - q0)
            lo = max(0, pos0 - window + 1) if window else 0
            want = -(-(hi - (lo // 128) * 128) // 128)
            pieces.sort()
            assert pieces[0][0] == 0 and sum(p[1] for p in pieces) == want
            for (a, an, _), (b, _, _) in zip(pieces, pieces[1:]):
                assert a + an == b
            assert (len(pieces) == 1) == (pieces[0][2] == -1)          # only cut rows have partial results
        assert sorted(seen) == sorted((i, q0) for i, s in enumerate(ctx.spans) if s.length >= 32
                                      for q0 in range(0, s.length, 128))
        assert nparts == sum(len(p) for p in seen.values() if len(p) > 1)
    # the adaptive piece: 6 heads x 43 tiles over 8 resident blocks is 33 tiles each, so pieces of the cap, 16
    ts, tq, n, cut = ctx.attention_items(32, 0, None, heads=6, slots=8)
    assert int(cut[1].max()) <= 16 and n == len(set(zip(ts.tolist(), tq.tolist(), cut[0].tolist())))


def test_layers_that_prepare_the_same_things_prepare_once(tmp_path):
    """Attention layers with equal heads, window and position encoding share one plan per step: only the first of
    them is called.  Tiny C has a full layer and two windowed ones, so two calls; tiny A one."""
    import json
    from lightllm_b200.config import load_config, model_spec_for
    from lightllm_b200.models.model import Model
    from tests.tiny_configs import config
    for name, want in (("A", 1), ("C", 2)):
        d = tmp_path / name
        d.mkdir()
        (d / "config.json").write_text(json.dumps(config(name)))
        model = Model(model_spec_for(load_config(str(d))))
        ctx = context([(0, 5, 0), (7, 1, 5)], staging_words=400)
        ctx.dtype, ctx.page_size, ctx.max_pages, ctx.decode_only, ctx.T = torch.float32, 16, 32, False, 6
        model.prepare(ctx, [None] * len(model.run))
        assert len(model._prepare_hooks) == want
        assert len([k for k in ctx.memo if k[0] == "attention_plan"]) == want


def test_every_span_of_a_mixed_step_goes_to_the_kernel_for_its_shape(tmp_path, monkeypatch):
    """The attention's plan for a step that mixes portions and tokens (no GPU: the kernels' own answers about what they
    support are asked, the device's SM count is given).  In bfloat16 with heads of 64: single tokens to the decode
    kernel, portions of two rows or more to the tensor-core kernel.  In float32: tiles of rows on CUDA cores, but few
    rows over many keys row by row with the keys in pieces."""
    import json
    from lightllm_b200.config import load_config, model_spec_for
    from lightllm_b200.csrc import ops
    from lightllm_b200.models.model import Model
    from lightllm_b200.parts import linear
    from tests.tiny_configs import config
    monkeypatch.setattr(linear, "num_sms", lambda device=None: 148)
    monkeypatch.setattr(ops, "decode_mma_cluster_splits", lambda: 16)
    d = tmp_path / "D"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(config("D")))
    mixer = Model(model_spec_for(load_config(str(d)))).layers[0].mixer          # layer 0 of D sees all keys
    spans = [(700, 1, 0), (600, 5, 1), (0, 100, 6), (0, 7, 106), (40, 1, 113)]

    def plan(dtype):
        ctx = context(spans, staging_words=4000)
        ctx.dtype, ctx.page_size, ctx.max_pages, ctx.decode_only, ctx.T = dtype, 16, 64, False, 114
        return mixer._plan(ctx, dtype)

    kind, items, decode, simt = plan(torch.bfloat16)
    assert kind == "mixed" and simt == []
    assert sorted(set(items[0].tolist())) == [1, 2, 3]                   # the portions, as items of the tensor-core kernel
    (tile_span, tile_q0, n), nsplit = decode
    assert tile_span.tolist() == [0, 4] and n == 2 and 1 <= nsplit <= 8  # the tokens, each request's keys in pieces
    kind, items, decode, simt = plan(torch.float32)
    assert items is None and decode is None and len(simt) == 2
    (rows_span, rows_q0, rows_n), bq, nsplit = simt[0]                   # few rows over many keys: row by row, in pieces
    assert bq == 1 and nsplit >= 2 and rows_span.tolist() == [0, 1, 1, 1, 1, 1] and rows_q0.tolist() == [0, 0, 1, 2, 3, 4]
    (tile_span, _, _), bq, nsplit = simt[1]                              # the rest in tiles of rows
    assert bq >= 1 and nsplit == 1 and sorted(set(tile_span.tolist())) == [2, 3, 4]


def test_a_mixed_step_described_row_by_row():
    """``rows_as_spans``: every token of every span becomes a span of one row at its own position, the rows keep their
    order (so an entry's wanted place is still its first row plus the place), and the last row is repeated up to a
    multiple of the bucket, never beyond the row limit."""
    from lightllm_b200.engine.batch import Span, rows_as_spans
    spans = [Span("a", 3, 40, 1, 0), Span("b", 5, 100, 4, 1), Span("c", 7, 0, 2, 5)]
    rows, firsts = rows_as_spans(spans, 8, 64)
    assert [(s.seq_id, s.start, s.length, s.row) for s in rows[:7]] == [
        ("a", 40, 1, 0), ("b", 100, 1, 1), ("b", 101, 1, 2), ("b", 102, 1, 3), ("b", 103, 1, 4), ("c", 0, 1, 5), ("c", 1, 1, 6)]
    assert [s.slot for s in rows[:7]] == [3, 5, 5, 5, 5, 7, 7]
    assert [(f.seq_id, f.row) for f in firsts] == [("a", 0), ("b", 1), ("c", 5)]
    assert len(rows) == 8 and (rows[7].seq_id, rows[7].start, rows[7].slot, rows[7].row) == ("c", 1, 7, 7)   # the padding
    rows, _ = rows_as_spans([Span("a", 0, 10, 16, 0)], 8, 64)
    assert len(rows) == 16                                   # already a multiple of the bucket: no padding
    rows, _ = rows_as_spans([Span("a", 0, 10, 61, 0)], 8, 62)
    assert len(rows) == 62 and all(r.start == 70 for r in rows[61:])      # the bucket stops at the row limit
