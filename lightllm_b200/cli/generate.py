"""``generate <model_dir> [token ids...]``: a prompt's continuation, in the manner of the
reference's tests/test_generate.cpp (prompt ids ``576 8319 315 13466 374``, 12 new tokens,
temperature 0.8, top-k 40, top-p 0.9; test_generate.cpp:148-149,284-290)."""
import argparse
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate")
    ap.add_argument("model_dir")
    ap.add_argument("tokens", nargs="*", type=int, default=[576, 8319, 315, 13466, 374])
    ap.add_argument("--max-new-tokens", type=int, default=12)
    ap.add_argument("--temperature", type=float, default=0.8)
    ap.add_argument("--top-k", type=int, default=40)
    ap.add_argument("--top-p", type=float, default=0.9)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--eos-token-id", type=int, default=None,
                    help="default: eos_token_id of the model's config.json (the reference fixes 151643, scheduler.h:29)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-seq-len", type=int, default=2048)
    args = ap.parse_args(argv)
    from lightllm_b200 import Engine
    eng = Engine(args.model_dir, dtype=args.dtype, max_seq_len=args.max_seq_len, max_seqs=4)
    prompt = [t % eng.vocab_size for t in args.tokens]
    out, why = eng.generate([prompt], args.max_new_tokens, args.temperature, args.top_k, args.top_p, args.min_p,
                            args.seed, args.eos_token_id, return_reasons=True)
    print("prompt:   ", " ".join(map(str, prompt)))
    print("generated:", " ".join(map(str, out[0])), f"({why[0]})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
