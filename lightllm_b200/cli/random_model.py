"""``random_model <config.json> <out_dir> [seed]``: write a model folder with random weights."""
import argparse
import json
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="random_model")
    ap.add_argument("config", help="a config.json of a known architecture")
    ap.add_argument("out_dir")
    ap.add_argument("seed", nargs="?", type=int, default=0)
    ap.add_argument("--store-dtype", default="bfloat16", choices=["bfloat16", "float32", "float16"])
    args = ap.parse_args(argv)
    from lightllm_b200 import write_random_model
    with open(args.config) as f:
        cfg = json.load(f)
    print(write_random_model(cfg, args.seed, args.out_dir, args.store_dtype))
    return 0


if __name__ == "__main__":
    sys.exit(main())
