"""The command lines run as a user runs them (``python -m lightllm_b200.cli...``), on a tiny model, and what they
print is checked against the plain implementation: the reference's tools drive its engine the same way
(tools/bench_server.cpp:158-245, tests/test_generate.cpp:284-290)."""
import os
import re
import subprocess
import sys

import pytest

from lightllm_b200.weights import write_random_model
from tests.plain import qwen2_plain as P
from tests.tiny_configs import config

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(module, *args):
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    proc = subprocess.run([sys.executable, "-m", module, *map(str, args)], stdout=subprocess.PIPE, stderr=subprocess.PIPE,
                          text=True, env=env, timeout=600, cwd=ROOT)
    assert proc.returncode == 0, proc.stderr[-3000:]
    return proc.stdout


@pytest.fixture(scope="module")
def tiny_a(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("cli_model"))
    write_random_model(config("A"), seed=3, out_dir=d, store_dtype="float32")
    return d, *P.read_model_dir(d)


def test_generate_prints_the_plain_greedy_continuation(tiny_a):
    d, cfg, w = tiny_a
    prompt = [5, 17, 3, 99, 250, 7]
    out = run_cli("lightllm_b200.cli.generate", d, *prompt, "--temperature", 0, "--max-new-tokens", 9, "--dtype", "float32",
                  "--max-seq-len", 64)
    got = re.search(r"generated:\s*([\d ]+)\((\w+)\)", out)
    assert got, out
    assert [int(t) for t in got.group(1).split()] == P.plain_greedy(cfg, w, prompt, 9)
    assert got.group(2) == "length"
    assert re.search(r"prompt:\s*5 17 3 99 250 7", out)


def test_generate_samples_the_same_tokens_for_the_same_seed(tiny_a):
    d, _, _ = tiny_a
    a = run_cli("lightllm_b200.cli.generate", d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64)
    b = run_cli("lightllm_b200.cli.generate", d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64)
    c = run_cli("lightllm_b200.cli.generate", d, 1, 2, 3, "--seed", 6, "--max-seq-len", 64)
    pick = lambda s: re.search(r"generated:\s*([\d ]+)", s).group(1)
    assert pick(a) == pick(b) != pick(c)
    assert len(pick(a).split()) == 12            # the reference's 12 new tokens (tests/test_generate.cpp:148-149)


def test_bench_server_runs_its_three_users_to_the_plain_tokens(tiny_a):
    d, cfg, w = tiny_a
    out = run_cli("lightllm_b200.cli.bench_server", d, 128, 64, "--dtype", "float32")
    V = cfg["vocab_size"]
    users = [([1, 2, 3, 4, 5], 15), (list(range(10, 30)), 10), ([7 * i % V for i in range(1, 41)], 20)]
    for i, (prompt, n) in enumerate(users):
        line = re.search(rf"\[user {i}\] \[([\d, ]+)\] \((\w+)\)", out)
        assert line, out
        assert [int(t) for t in line.group(1).split(",")] == P.plain_greedy(cfg, w, [t % V for t in prompt], n)
        assert line.group(2) == "length"
    assert re.search(r"Total tokens: 45 ", out) and "steps/s" in out
    steps = re.findall(r"\[step\s+\d+\] tokens=\s*(\d+) prefill=\s*(\d+) decode=\s*(\d+)", out)
    assert steps and all(int(t) == int(p) + int(dd) and int(t) <= 64 for t, p, dd in steps)


def test_random_model_writes_a_folder_the_engine_loads(tmp_path):
    import json
    cfg_path = str(tmp_path / "config.json")
    with open(cfg_path, "w") as f:
        json.dump(config("B"), f)
    out_dir = str(tmp_path / "made")
    run_cli("lightllm_b200.cli.random_model", cfg_path, out_dir, 4)
    assert sorted(os.listdir(out_dir)) == ["config.json", "model.safetensors"]
    text = run_cli("lightllm_b200.cli.generate", out_dir, 1, 2, 3, "--temperature", 0, "--max-new-tokens", 3, "--max-seq-len", 64)
    assert re.search(r"generated:\s*\d+ \d+ \d+", text)


def test_bench_ops_times_every_operator():
    """The operator benchmark at small sizes: every operator reports a time and the bytes it moves."""
    import json
    out = run_cli("lightllm_b200.cli.bench_ops", "--rows", 64, "--batch", 3, "--context", 200, "--reps", 2, "--hidden", 128,
                  "--heads", 4, "--kv-heads", 2, "--head-dim", 64, "--intermediate", 256, "--vocab", 9001)
    recs = [json.loads(line) for line in out.splitlines() if line.startswith("{")]
    names = [r["op"] for r in recs]
    for want in ("embedding", "rmsnorm", "rmsnorm_float32", "rope_table", "rope_kv_write", "gemm_simt_float32",
                 "paged_attention_simt_float32", "paged_attention_tcgen05", "paged_decode_mma",
                 "paged_decode_mma_and_merge", "argmax", "sample_top_k_top_p", "sample_temperature_only", "mma_issue"):
        assert want in names, names
    assert all(r["us"] > 0 and r["MB"] > 0 for r in recs if r["op"] != "mma_issue")
    assert all(r["cycles_per_mma"] > 0 for r in recs if r["op"] == "mma_issue")


# ---- the C++ generate program (csrc/host/generate.cpp) -------------------------------------------------------------------
def run_cpp_generate(*args, ok=True):
    from lightllm_b200.csrc.build import tool_path
    proc = subprocess.run([tool_path(), *map(str, args)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=600)
    assert (proc.returncode == 0) == ok, proc.stderr[-3000:]
    return proc.stdout if ok else proc.stderr


def cpp_outputs(text):
    return [(list(map(int, m.group(1).split())), m.group(2)) for m in re.finditer(r"generated:\s*([\d ]+)\((\w+)\)", text)]


@pytest.mark.parametrize("name", ["E", "D"])
def test_cpp_generate_follows_the_plain_implementation(tmp_path, name):
    """Three prompts through the C++ program, with a token budget that cuts the longer prompts into portions which run
    beside the decoded tokens of the requests that started earlier: every token is the plain implementation's choice
    for the same history.  E has heads of 128 and an untied head; D (without its window) heads of 64 in groups of 3
    and a tied head."""
    import random
    from tests.test_engine_gpu import assert_greedy_follows_plain
    cfg = config(name)
    cfg["use_sliding_window"] = False
    d = str(tmp_path / "m")
    write_random_model(cfg, seed=11, out_dir=d, store_dtype="bfloat16")
    cfg, w = P.read_model_dir(d)
    rng = random.Random(4)
    prompts = [[rng.randrange(cfg["vocab_size"]) for _ in range(n)] for n in (5, 300, 139)]
    args = []
    for p in prompts:
        args += p + ["/"]
    out = run_cpp_generate(d, *args[:-1], "--temperature", 0, "--max-new-tokens", 20, "--eos-token-id", 100000,
                           "--max-batch-tokens", 128, "--max-seq-len", 512)
    got = cpp_outputs(out)
    assert [why for _, why in got] == ["length"] * 3
    assert all(len(o) == 20 for o, _ in got)
    assert_greedy_follows_plain(cfg, w, prompts, [o for o, _ in got], name, "bfloat16")
    # and the Python entry point, which runs the same kernels over the same cuts of the layers, says the same
    from lightllm_b200 import Engine
    eng = Engine(d, dtype="bfloat16", max_seq_len=512, max_batch_tokens=128, max_seqs=4)
    ref = eng.generate(prompts, max_new_tokens=20, temperature=0.0, eos_token_id=-1)
    same = sum(a == b for (o, _), r in zip(got, ref) for a, b in zip(o, r))
    assert same >= 54, (got, ref)          # a near-tie may fall the other way where the two cut their steps differently


def test_cpp_generate_samples_the_same_tokens_for_the_same_seed(tmp_path):
    d = str(tmp_path / "m")
    write_random_model(config("E"), seed=3, out_dir=d, store_dtype="bfloat16")
    a = cpp_outputs(run_cpp_generate(d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64))
    b = cpp_outputs(run_cpp_generate(d, 1, 2, 3, "--seed", 5, "--max-seq-len", 64))
    c = cpp_outputs(run_cpp_generate(d, 1, 2, 3, "--seed", 6, "--max-seq-len", 64))
    assert a == b and a != c
    assert len(a[0][0]) == 12 or a[0][1] == "eos"          # the reference's 12 new tokens (tests/test_generate.cpp:148-149)
    # top-k of one leaves the sampler no choice: the greedy tokens, whatever the temperature and the seed
    greedy = cpp_outputs(run_cpp_generate(d, 1, 2, 3, "--temperature", 0, "--max-seq-len", 64, "--eos-token-id", 100000))
    forced = cpp_outputs(run_cpp_generate(d, 1, 2, 3, "--temperature", 1.5, "--top-k", 1, "--seed", 9, "--max-seq-len", 64,
                                          "--eos-token-id", 100000))
    assert greedy == forced and len(greedy[0][0]) == 12
    # a long prompt that ends at the sequence limit
    long = cpp_outputs(run_cpp_generate(d, *range(1, 60), "--temperature", 0, "--max-seq-len", 64, "--eos-token-id", 100000))
    assert long[0][1] == "max_seq_len" and len(long[0][0]) == 5
