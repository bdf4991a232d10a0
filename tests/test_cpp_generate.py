"""What the C++ ``generate`` program (csrc/host/generate.cpp) says before it touches a device: its reading of
config.json and model.safetensors and of its own command line.  The program is compiled with the kernel library."""
import json
import os
import shutil
import subprocess

import pytest

from lightllm_b200.weights import write_random_model
from tests.tiny_configs import config

pytestmark = pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"),
                                reason="nvcc is needed to build the program")


def run(*args):
    from lightllm_b200.csrc.build import tool_path
    proc = subprocess.run([tool_path(), *map(str, args)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=900)
    return proc.returncode, proc.stdout, proc.stderr


@pytest.fixture(scope="module")
def model_e(tmp_path_factory):
    d = str(tmp_path_factory.mktemp("cpp_model"))
    write_random_model(config("E"), seed=1, out_dir=d, store_dtype="bfloat16")
    return d


def rewrite(model_dir, tmp_path, **changes):
    d = str(tmp_path / "changed")
    shutil.copytree(model_dir, d)
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    cfg.update(changes)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    return d


def test_one_error_lists_what_is_wrong_with_the_weights(model_e, tmp_path):
    d = rewrite(model_e, tmp_path, intermediate_size=528, tie_word_embeddings=True)
    rc, _, err = run(d, 1, 2, 3)
    assert rc == 1
    assert "does not fit config.json" in err
    assert "model.layers.0.mlp.gate_proj.weight has shape [520, 256], expected [528, 256]" in err
    assert "model.layers.1.mlp.down_proj.weight has shape [256, 520], expected [256, 528]" in err
    assert "missing" not in err                      # a tied head reads the embedding; lm_head.weight is then ignored
    d2 = rewrite(model_e, tmp_path / "x", num_hidden_layers=3)
    rc, _, err = run(d2, 1)
    assert rc == 1 and "missing tensors (12)" in err and "model.layers.2.self_attn.q_proj.bias" in err


def test_configurations_it_does_not_run_name_the_python_entry_point(model_e, tmp_path):
    d = rewrite(model_e, tmp_path, use_sliding_window=True, sliding_window=64, max_window_layers=1)
    rc, _, err = run(d, 1, 2)
    assert rc == 1 and "sliding window" in err and "lightllm_b200.cli.generate" in err
    d = rewrite(model_e, tmp_path / "y", architectures=["LlamaForCausalLM"])
    rc, _, err = run(d, 1, 2)
    assert rc == 1 and "LlamaForCausalLM" in err
    d = rewrite(model_e, tmp_path / "z", head_dim=48, num_attention_heads=4)
    rc, _, err = run(d, 1, 2)
    assert rc == 1 and "heads of 48" in err


def test_config_errors_name_the_key(model_e, tmp_path):
    d = rewrite(model_e, tmp_path, vocab_size=None)
    rc, _, err = run(d)
    assert rc == 1 and "required key 'vocab_size' is missing" in err
    d = rewrite(model_e, tmp_path / "a", rms_norm_eps="small")
    rc, _, err = run(d)
    assert rc == 1 and "'rms_norm_eps' must be a number" in err
    with open(os.path.join(d, "config.json"), "w") as f:
        f.write('{"architectures": ["Qwen2ForCausalLM"], ')
    rc, _, err = run(d)
    assert rc == 1 and "not valid JSON" in err


def test_command_line_errors(model_e):
    assert "unknown option --bogus" in run(model_e, "--bogus")[2]
    assert "an empty prompt before '/'" in run(model_e, "/", 1)[2]
    assert "needs a value" in run(model_e, 1, "--seed")[2]
    assert "bfloat16 only" in run(model_e, 1, "--dtype", "float32")[2]
    rc, out, _ = run("--help")
    assert rc == 0 and "--max-new-tokens" in out
    # without a device (the tests that are not marked gpu run where there is none) it says so after all checks passed
    rc, _, err = run(model_e, 1, 2, 3)
    assert rc == 0 or "no CUDA device" in err or "sm_100a" in err


def test_its_attention_items_are_cut_as_the_engine_cuts_them():
    """The program plans the tensor-core attention's work items itself; for the same row tiles, heads and resident
    blocks it must choose the piece length and produce the items, merges and parts that ``engine/batch.py`` does."""
    import random
    from lightllm_b200.engine.batch import cut_attention_rows
    rng = random.Random(0)
    cases = [[16], list(range(1, 17)), list(range(1, 65)), [3, 40, 2, 9], [64] * 5]
    cases += [[rng.randrange(1, 70) for _ in range(rng.randrange(1, 40))] for _ in range(12)]
    for tiles in cases:
        for heads, slots in ((14, 296), (12, 148), (28, 148), (2, 37)):
            rows = [(0, 128 * i, n) for i, n in enumerate(tiles)]
            items, merges, parts = cut_attention_rows(rows, None, heads, slots)
            rc, out, err = run("--cut-rows", " ".join(map(str, tiles)), heads, slots)
            assert rc == 0, err
            got_items = [tuple(map(int, l.split()[1:])) for l in out.splitlines() if l.startswith("item")]
            got_merges = [tuple(map(int, l.split()[1:])) for l in out.splitlines() if l.startswith("merge")]
            got_parts = int(out.splitlines()[-1].split()[1])
            assert got_items == [tuple(t) for t in items], (tiles, heads, slots)
            assert got_merges == [tuple(m) for m in merges] and got_parts == parts
