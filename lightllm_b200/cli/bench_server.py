"""``bench_server <model_dir> [max_seq_len] [max_batch_tokens]`` (tools/bench_server.cpp:33-43).

Three fixed users through the DecodeFirst scheduler with ``chunk_size=16``: prints every
generated token, then tokens a second and steps a second (bench_server.cpp:158-245).  Extra
options of this engine come after the positional ones: ``--dtype``, ``--temperature``.
"""
import argparse
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bench_server", usage="bench_server <model_dir> [max_seq_len] [max_batch_tokens]")
    ap.add_argument("model_dir")
    ap.add_argument("max_seq_len", nargs="?", type=int, default=2048)
    ap.add_argument("max_batch_tokens", nargs="?", type=int, default=256)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--temperature", type=float, default=0.0)
    args = ap.parse_args(argv)

    from lightllm_b200 import Engine
    print("=" * 60)
    print("  LightLLM-B200 Scheduler-Engine Benchmark")
    print("=" * 60)
    print(f"  Model dir:      {args.model_dir}")
    print(f"  Max seq len:    {args.max_seq_len}")
    print(f"  Max batch tok:  {args.max_batch_tokens}")
    print("  Scheduler:      DecodeFirst (chunk_size=16)")
    print("=" * 60)
    print("[init] Loading model...")
    eng = Engine(args.model_dir, dtype=args.dtype, max_seq_len=args.max_seq_len,
                 max_batch_tokens=args.max_batch_tokens, chunk_size=16, max_seqs=8)
    spec = eng.core.model.spec
    print(f"[init] Model loaded. Hidden dim={spec.hidden_size}, vocab={spec.vocab_size}, layers={len(spec.layers)}")
    V = spec.vocab_size
    users = [([1, 2, 3, 4, 5], 15), (list(range(10, 30)), 10), ([7 * i % V for i in range(1, 41)], 20)]
    loop = eng.new_loop()
    ids = [loop.submit([t % V for t in p], max_new_tokens=n, temperature=args.temperature)
           for p, n in users]
    t0 = time.perf_counter()
    shown = 0

    def show():           # a step's figures are known once its ids have been read, one step later while steps overlap
        nonlocal shown
        for m in loop.step_metrics[shown:]:
            print(f"[step {m.step_number:3d}] tokens={m.tokens_processed:3d} prefill={m.prefill_tokens:3d} "
                  f"decode={m.decode_tokens:2d} active={m.active_after}")
        shown = len(loop.step_metrics)
    while loop.has_active():
        loop.step()
        show()
    loop.flush()
    show()
    dt = time.perf_counter() - t0
    for i in ids:
        print(f"[user {i}] {loop.generated_tokens(i)} ({loop.finish_reason(i)})")
    total = loop.total_tokens_generated()
    print(f"Total tokens: {total}  time: {dt:.3f} s  throughput: {total / dt:.1f} tok/s  "
          f"steps/s: {loop.total_steps / dt:.1f}")
    print(f"P50 TTFT {loop.stat('ttft', 50):.1f} ms  P50 TPOT {loop.stat('tpot', 50):.2f} ms  "
          f"P50 latency {loop.stat('latency', 50):.1f} ms")
    return 0


if __name__ == "__main__":
    sys.exit(main())
