#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode tokens a second at Qwen2.5-0.5B sizes.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L]
    python bench.py --sizes 1.5b|7b          (the larger sizes of the family: a line of their own)
    python bench.py [--sizes ..] --only decode|prefill [--prompt-len N]     (one part, at another context length)
    python bench.py --only small-mixed       (the steps of a loaded server: a 16-token portion beside decoded tokens)

Prints one JSON line.  ``value`` is decoded tokens a second over K timed decode steps of a
batch of 8 requests that each hold a 2,048-token prompt (random weights, random token ids),
timed on the device with CUDA events.  ``e2e`` is the same through the Python entry point's
serve loop, with host token ids in and out every step.  ``prefill`` is one 2,048-token prompt
in one step; ``points`` are decode at batch 1 and 64; ``roofline`` relates the decode step to
the bytes it has to read.  The engine runs on one GPU only: for ``--gpus`` above 1 it says so
and exits with 2.  ``--impl reference`` reports why the reference cannot run here.
"""
import argparse
import json
import os
import random
import shutil
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# BASELINE.json configs[2]: Qwen2.5-0.5B sizes.
QWEN25_05B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 24, "hidden_size": 896, "num_attention_heads": 14, "num_key_value_heads": 2,
    "intermediate_size": 4864, "vocab_size": 151936, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 32768, "sliding_window": 32768,
    "max_window_layers": 24, "use_sliding_window": False, "hidden_act": "silu",
}
# The larger sizes BASELINE.json lists (its configs[3] and configs[4]), measured with `--sizes`.
QWEN25_15B = dict(QWEN25_05B, num_hidden_layers=28, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2,
                  head_dim=128, intermediate_size=8960, max_window_layers=28)
QWEN25_7B = dict(QWEN25_05B, num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4,
                 head_dim=128, intermediate_size=18944, vocab_size=152064, tie_word_embeddings=False, max_window_layers=28)
SIZES = {"0.5b": QWEN25_05B, "1.5b": QWEN25_15B, "7b": QWEN25_7B}
PROMPT_LEN = 2048
CONTEXT_LEN = 4096
PAGE_SIZE = 16


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        exe = shutil.which("nvidia-smi")
        if not exe:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.proc = subprocess.Popen([exe, "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) == 6 and parts[0].isdigit():
                    rows.append(parts)
        os.remove(self.path)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[2 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def make_model_dir(layers: int) -> str:
    from lightllm_b200 import write_random_model
    cfg = dict(QWEN25_05B)
    cfg["num_hidden_layers"] = layers
    cfg["max_window_layers"] = layers
    d = tempfile.mkdtemp(prefix="llb_bench_model_")
    write_random_model(cfg, seed=0, out_dir=d, store_dtype="bfloat16")
    return d


def flops_prefill(cfg, layers, T):
    D, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]
    hd = cfg.get("head_dim", D // Hq)
    linear = 2 * T * (D * (Hq + 2 * Hkv) * hd + Hq * hd * D + 3 * D * I)
    attn = 2 * 2 * Hq * hd * T * (T + 1) // 2      # QK^T and PV over the causal half
    return layers * (linear + attn) + 2 * D * V    # head for the last row


def decode_bytes(core, batch, ctx_len):
    """Bytes a decode step has to read: every weight it uses once, and the cache of the live requests."""
    esize = 2
    kv = core.model.cache_layout.bytes_per_token(esize) * batch * ctx_len
    weights = core.model.weight_bytes()
    D, V = core.model.spec.hidden_size, core.model.spec.vocab_size
    # the embedding table is the head's matrix when tied and is then read in full; rows gathered are negligible
    if core.model.head.weight.data_ptr() != core.model.embedding.table.data_ptr():
        weights -= V * D * esize
    return weights + kv


def time_decode(core, batch, steps, warmup, rng, clocks=None):
    import torch
    from lightllm_b200.engine import StepEntry
    V = core.vocab_size
    ids = list(range(batch))
    for i in ids:
        core.open(i)
    # prefill every request's 2,048-token prompt (a few requests a step)
    per_step = max(1, core.runner.max_batch_tokens // PROMPT_LEN)
    for a in range(0, batch, per_step):
        core.step([StepEntry(i, [rng.randrange(V) for _ in range(PROMPT_LEN)], []) for i in ids[a:a + per_step]])
    def one():
        return core.step([StepEntry(i, [rng.randrange(V)], [0]) for i in ids])
    for _ in range(warmup):
        one()
    torch.cuda.synchronize()
    if clocks is not None:
        clocks.start()
        time.sleep(0.12)          # let the sampler take its first reading before the timed region
    l0 = core.launch_count()
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        one()
    t1.record()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1) / steps
    launches = core.launch_count() - l0
    ctx = PROMPT_LEN + warmup + steps // 2
    for i in ids:
        core.close(i)
    return ms, launches, ctx


def time_prefill(core, steps, warmup, rng):
    import torch
    from lightllm_b200.engine import StepEntry
    V = core.vocab_size
    times = []
    for it in range(warmup + steps):
        core.open("p")
        toks = [rng.randrange(V) for _ in range(PROMPT_LEN)]
        torch.cuda.synchronize()
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        core.step([StepEntry("p", toks, [PROMPT_LEN - 1])])
        t1.record()
        torch.cuda.synchronize()
        if it >= warmup:
            times.append(t0.elapsed_time(t1))
        core.close("p")
    return sum(times) / len(times)


def time_e2e(engine, batch, steps, warmup, rng):
    """Decode through the public serve loop: host token ids in, sampled ids out, every step."""
    import torch
    V = engine.vocab_size
    loop = engine.new_loop()
    for _ in range(batch):
        loop.submit([rng.randrange(V) for _ in range(PROMPT_LEN)], max_new_tokens=warmup + steps + 8,
                    eos_token_id=-1, temperature=0.0)
    while any(r.state != "DECODING" for r in loop.scheduler.running) or loop.scheduler.waiting:
        loop.step()
    for _ in range(warmup):
        loop.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        loop.step()
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    h2d = engine.core.runner.last_h2d_bytes
    for r in list(loop.scheduler.running):
        loop.scheduler.finish_request(r.id)
    return batch * steps / dt, h2d, 4 * batch


def time_mixed(engine, requests, lo, hi, new_tokens, rng):
    """BASELINE.json configs[3]'s workload through the serve loop: `requests` prompts with lengths uniform in
    [lo, hi], all submitted at once, prompt portions under the loop's token budget beside decoded tokens,
    `new_tokens` tokens each (the reference measures the same way, tools/bench_mixed_lengths.cpp)."""
    import torch
    V = engine.vocab_size
    loop = engine.new_loop()
    loop.measure_device = True
    lens = [rng.randint(lo, hi) for _ in range(requests)]
    for n in lens:
        loop.submit([rng.randrange(V) for _ in range(n)], max_new_tokens=new_tokens, eos_token_id=-1, temperature=0.0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    loop.run()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    busy = loop.device_busy_ms() / 1000.0
    steps = loop.step_metrics
    return {"requests": requests, "prompt_tokens": sum(lens), "generated": loop.total_tokens_generated(),
            "steps": len(steps), "seconds": round(wall, 3),
            "generated_tok_s": round(loop.total_tokens_generated() / wall, 1),
            "all_tok_s": round((sum(lens) + loop.total_tokens_generated()) / wall, 1),
            "ms_per_step": round(1000.0 * wall / max(1, len(steps)), 3),
            "host_share": round(max(0.0, 1.0 - busy / wall), 3),
            "ttft_ms_p50": round(loop.stat("ttft", 50), 1), "tpot_ms_p50": round(loop.stat("tpot", 50), 2)}


def time_small_mixed(core, steps, warmup, rng, portion=16, decoders=20):
    """Steps as a loaded server runs them: one `portion`-token piece of a prompt beside the decoded tokens of 1 to 16
    of `decoders` requests (contexts of a few hundred to a few thousand tokens), a different composition every step.
    Milliseconds a step, host and device together (the steps are issued back to back and awaited after every hundred;
    the median hundred is reported)."""
    import torch
    from lightllm_b200.engine import StepEntry
    V = core.vocab_size
    n = decoders + 4
    for i in range(n):
        core.open(i)
        core.step([StepEntry(i, [rng.randrange(V) for _ in range(300 + 37 * i)], [0])])

    held = {i: 300 + 37 * i for i in range(n)}
    limit = core.runner.max_pages * core.cache.page_size - 64

    def run(count):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for s in range(count):
            who = rng.sample(range(decoders), rng.randrange(1, 17))
            pre = decoders + s % 4
            for i in who + [pre]:
                if held[i] + portion > limit:          # a request that has grown to the limit starts over
                    core.close(i)
                    core.open(i)
                    held[i] = 0
            entries = [StepEntry(i, [rng.randrange(V)], [0]) for i in who]
            entries.append(StepEntry(pre, [rng.randrange(V) for _ in range(portion)], []))
            core.step(entries)
            for i in who:
                held[i] += 1
            held[pre] += portion
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / count * 1e3
    run(warmup)
    blocks = sorted(run(100) for _ in range(max(1, steps // 100)))      # the median block: the host's noise stays out
    for i in range(n):
        core.close(i)
    return blocks[len(blocks) // 2]


def run_sizes(name: str, steps: int, warmup: int, layers=None, only=None) -> int:
    """Decode at batch 1 / 8 / 64 and a 2,048-token prefill at one of the larger sizes, with their roofline
    fractions, and for the 1.5B sizes the mixed workload.  Weights are drawn on the device."""
    import torch
    from lightllm_b200 import Engine
    from lightllm_b200.models import random_model_on_device
    cfg = dict(SIZES[name])
    layers_of_config = cfg["num_hidden_layers"]
    if layers:               # fewer layers of the same sizes (for profiling runs); both numbers are reported
        cfg["num_hidden_layers"] = cfg["max_window_layers"] = layers
    pk = peaks()
    rng = random.Random(0)
    device = torch.device("cuda:0")
    torch.cuda.set_device(device)
    model = random_model_on_device(dict(cfg), 0, "bfloat16", device)
    max_batch = 64
    engine = Engine(None, dtype="bfloat16", max_seq_len=CONTEXT_LEN + 512, max_batch_tokens=4 * PROMPT_LEN, page_size=PAGE_SIZE,
                    num_pages=max_batch * (PROMPT_LEN + 512) // PAGE_SIZE, max_seqs=max_batch, chunk_size=PROMPT_LEN,
                    model=model)
    core = engine.core
    out = {"sizes": name, "dtype": "bf16", "data": "synthetic: random weights drawn on the device (seed 0)",
           "config": {"layers": cfg["num_hidden_layers"], "layers_of_config": layers_of_config, "hidden": cfg["hidden_size"],
                      "heads": cfg["num_attention_heads"],
                      "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg.get("head_dim", 64),
                      "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                      "tied_embeddings": cfg["tie_word_embeddings"], "prompt_len": PROMPT_LEN, "page_size": PAGE_SIZE},
           "peaks": pk["source"], "decode": {}}
    for b in (() if only == "prefill" else (1, 8, 64)):
        ms, _, ctx = time_decode(core, b, steps, warmup, rng)
        gbs = decode_bytes(core, b, ctx) / (ms * 1e-3) / 1e9
        out["decode"][f"b{b}"] = {"tok_s": round(b * 1000.0 / ms, 1), "ms_per_step": round(ms, 4), "gb_s": round(gbs, 1),
                                  "frac_of_hbm": round(gbs / pk["hbm_gbs"], 4)}
    if only == "decode":
        print(json.dumps(out))
        return 0
    pre_ms = time_prefill(core, 4 if only is None else steps, 3, rng)
    fl = flops_prefill(cfg, cfg["num_hidden_layers"], PROMPT_LEN)
    out["prefill"] = {"tok_s": round(PROMPT_LEN * 1000.0 / pre_ms, 1), "ms": round(pre_ms, 3),
                      "frac_of_bf16_peak": round(fl / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
    if name == "1.5b" and only is None:
        del engine, core
        mixed = Engine(None, dtype="bfloat16", max_seq_len=4096 + 128 + 16, max_batch_tokens=2048, page_size=PAGE_SIZE,
                       num_pages=32 * (4096 + 256) // PAGE_SIZE, max_seqs=32, chunk_size=2048, model=model)
        out["mixed"] = time_mixed(mixed, 32, 64, 4096, 128, rng)
    print(json.dumps(out))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=QWEN25_05B["num_hidden_layers"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="only the headline batch (for profiling runs)")
    ap.add_argument("--sizes", choices=["1.5b", "7b"], default=None,
                    help="measure at the Qwen2.5-1.5B or 7B layer sizes instead (a line of its own, not the bench record)")
    ap.add_argument("--prompt-len", type=int, default=None,
                    help="tokens each request holds before decoding starts (default 2,048); with --only or --sizes, for "
                         "measurements at other context lengths, not for the bench record")
    ap.add_argument("--only", choices=["decode", "prefill", "small-mixed"], default=None,
                    help="run one part only and print a short line (for profiling runs, not a bench record)")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "the reference is a C++/CMake project without setup.py or pyproject.toml (pip: 'not "
                          "installable'), and its build needs the absent third_party/xgrammar submodule"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(3, args.warmup)
    if args.prompt_len:
        if not (args.only or args.sizes) or args.prompt_len < 16:
            print("bench.py: --prompt-len goes with --only or --sizes and is at least 16")
            return 2
        global PROMPT_LEN, CONTEXT_LEN
        PROMPT_LEN, CONTEXT_LEN = args.prompt_len, args.prompt_len + 2048
    if args.sizes:
        return run_sizes(args.sizes, min(args.steps, 64), args.warmup,
                         args.layers if args.layers != QWEN25_05B["num_hidden_layers"] else None, args.only)

    import torch
    from lightllm_b200 import Engine
    rng = random.Random(0)
    pk = peaks()
    model_dir = make_model_dir(args.layers)
    try:
        max_batch = 64
        engine = Engine(model_dir, dtype="bfloat16", max_seq_len=CONTEXT_LEN, max_batch_tokens=4 * PROMPT_LEN,
                        page_size=PAGE_SIZE, num_pages=max_batch * (PROMPT_LEN + 512) // PAGE_SIZE,
                        max_seqs=max_batch, chunk_size=PROMPT_LEN)
        core = engine.core
        if args.only == "decode":
            ms, launches, ctx = time_decode(core, args.batch, args.steps, args.warmup, rng)
            r = core.runner
            extra = {"graph_replays": r.graph_replays, "graphs": len(r._graphs)}
            if r._graphs:      # the same captured step replayed back to back: device time without any host work
                g = next(iter(r._graphs.values()))[0]
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(20):
                    g.replay()
                e1.record()
                torch.cuda.synchronize()
                extra["replay_only_ms"] = round(e0.elapsed_time(e1) / 20, 4)
            gbs = decode_bytes(core, args.batch, ctx) / (ms * 1e-3) / 1e9
            print(json.dumps({"only": "decode", "batch": args.batch, "context": ctx, "ms_per_step": round(ms, 4),
                              "gb_s": round(gbs, 1), "frac_of_hbm": round(gbs / pk["hbm_gbs"], 4), "launches": launches,
                              **extra}))
            return 0
        if args.only == "small-mixed":
            ms = time_small_mixed(core, min(args.steps, 600), 150, rng)
            r = core.runner
            print(json.dumps({"only": "small-mixed", "ms_per_step": round(ms, 4), "row_by_row": bool(r.rowwise),
                              "graph_replays": r.graph_replays, "graphs": len(r._graphs)}))
            return 0
        if args.only == "prefill":
            pre_ms = time_prefill(core, args.steps, args.warmup, rng)
            fl = flops_prefill(QWEN25_05B, args.layers, PROMPT_LEN)
            print(json.dumps({"only": "prefill", "tokens": PROMPT_LEN, "ms": round(pre_ms, 3),
                              "frac_of_bf16_peak": round(fl / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}))
            return 0
        args.steps = min(args.steps, 448)        # the pool holds 2,048 + 512 tokens per request
        clocks = ClockSampler()
        ms, launches, ctx = time_decode(core, args.batch, args.steps, args.warmup, rng, clocks)
        clk = clocks.stop()
        value = args.batch * 1000.0 / ms
        achieved = decode_bytes(core, args.batch, ctx) / (ms * 1e-3) / 1e9
        e2e_value, h2d, d2h = time_e2e(engine, args.batch, args.steps, args.warmup, rng)
        pre_ms = time_prefill(core, 5, 3, rng)
        fl = flops_prefill(QWEN25_05B, args.layers, PROMPT_LEN)
        points = {}
        if not args.skip_points:
            for b in (1, 64):
                pms, _, _ = time_decode(core, b, args.steps, args.warmup, rng)
                points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
        cfg = QWEN25_05B
        line = {
            "metric": "decode tok/s at batch 8 (Qwen2.5-0.5B sizes, 2,048-token prompts)",
            "value": round(value, 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic: random weights (seed 0), token ids uniform in vocab",
            "config": {
                "model": "Qwen2.5-0.5B sizes (Qwen2ForCausalLM)", "global_batch": args.batch, "seq_len": CONTEXT_LEN,
                "prompt_len": PROMPT_LEN, "parallelism": "single GPU", "layers": args.layers,
                "layers_of_config": cfg["num_hidden_layers"], "hidden": cfg["hidden_size"],
                "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"], "intermediate": cfg["intermediate_size"],
                "vocab": cfg["vocab_size"], "page_size": PAGE_SIZE, "tied_embeddings": cfg["tie_word_embeddings"],
                "l2": "inputs larger than L2: the weights read every step are ~1 GB",
                "peaks": pk["source"],
            },
            "e2e": {"value": round(e2e_value, 1), "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches,
            "clocks": clk,
            "prefill": {"value": round(PROMPT_LEN * 1000.0 / pre_ms, 1), "tokens": PROMPT_LEN, "ms": round(pre_ms, 3),
                        "frac": round(fl / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)},
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
            "points": points,
        }
        print(json.dumps(line))
    finally:
        shutil.rmtree(model_dir, ignore_errors=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
