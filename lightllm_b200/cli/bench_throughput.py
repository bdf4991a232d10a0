"""``bench_throughput <model_dir> [duration_sec] [arrival_rate]`` (tools/bench_throughput.cpp:33-35).

Poisson arrivals at ``arrival_rate`` requests a second for ``duration_sec`` seconds; prompts are
short, medium or long with probabilities 50/35/15 % (bench_throughput.cpp:43-60, as random token
ids here); ``CHUNK_SIZE=16``, ``MAX_BATCH_TOKENS=512``.  Prints TTFT, TPOT and latency
percentiles and tokens a second at the end."""
import argparse
import random
import sys
import time


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="bench_throughput")
    ap.add_argument("model_dir")
    ap.add_argument("duration_sec", nargs="?", type=float, default=60.0)
    ap.add_argument("arrival_rate", nargs="?", type=float, default=1.0)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-seq-len", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=1)
    args = ap.parse_args(argv)
    from lightllm_b200 import Engine
    eng = Engine(args.model_dir, dtype=args.dtype, max_seq_len=args.max_seq_len, max_batch_tokens=512, chunk_size=16)
    loop = eng.new_loop()
    rng = random.Random(args.seed)
    V = eng.vocab_size
    t0 = time.perf_counter()
    next_arrival = 0.0
    while True:
        now = time.perf_counter() - t0
        while now >= next_arrival and next_arrival < args.duration_sec:
            u = rng.random()
            plen, new = (rng.randint(8, 32), 32) if u < 0.5 else (rng.randint(64, 160), 64) if u < 0.85 \
                else (rng.randint(256, 512), 128)
            loop.submit([rng.randrange(V) for _ in range(plen)], max_new_tokens=new, eos_token_id=-1, temperature=0.0)
            next_arrival += rng.expovariate(args.arrival_rate)
        if not loop.step():
            if next_arrival >= args.duration_sec:
                break
            time.sleep(min(0.005, max(0.0, next_arrival - now)))
    dt = time.perf_counter() - t0
    done = [m for m in loop.all_metrics() if m.finished]
    print(f"requests finished: {len(done)}  tokens: {loop.total_tokens_generated()}  "
          f"throughput: {loop.total_tokens_generated() / dt:.1f} tok/s  steps: {loop.total_steps}")
    for what in ("ttft", "tpot", "latency"):
        print(f"{what.upper():8s} avg {loop.stat(what):9.2f} ms  " +
              "  ".join(f"P{p} {loop.stat(what, p):9.2f}" for p in (50, 90, 95, 99)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
