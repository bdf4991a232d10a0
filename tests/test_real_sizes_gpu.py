"""The engine at the real layer sizes of the benchmark model (hidden 896, 14 query heads in 2 groups of 7, head 64,
intermediate 4864, vocabulary 151936, tied head), with two layers and random weights, against the plain implementation:
whole prompt, portions beside decoded tokens, and one-by-one decoding (graph replay included), in both precisions.
This is where the tensor-core kernels run at the shapes they were written for."""
import random

import pytest
import torch

from lightllm_b200 import EngineCore, EngineOptions, StepEntry, write_random_model
from tests.plain.qwen2_plain import plain_forward, read_model_dir
from tests.tolerances import atol_for, logits_std, record

pytestmark = pytest.mark.gpu

REAL = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "num_hidden_layers": 2, "hidden_size": 896,
    "num_attention_heads": 14, "num_key_value_heads": 2, "intermediate_size": 4864, "vocab_size": 151936,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 32768,
    "use_sliding_window": False, "hidden_act": "silu",
}


@pytest.fixture(scope="module")
def real_model(tmp_path_factory):
    out = {}
    for store in ("float32", "bfloat16"):
        d = str(tmp_path_factory.mktemp(f"real_{store}"))
        write_random_model(dict(REAL), seed=21, out_dir=d, store_dtype=store)
        cfg, w = read_model_dir(d)
        rng = random.Random(5)
        seqs = {"a": [rng.randrange(151936) for _ in range(300)], "b": [rng.randrange(151936) for _ in range(45)]}
        ref = {k: plain_forward(cfg, w, v) for k, v in seqs.items()}
        out[store] = (d, seqs, ref)
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_real_sizes_whole_portions_and_decode(real_model, dtype):
    d, seqs, ref = real_model["float32" if dtype == "float32" else "bfloat16"]
    core = EngineCore(d, EngineOptions(dtype=dtype, max_seq_len=512, max_batch_tokens=512, page_size=16,
                                       num_pages=48, max_seqs=4))
    tol = atol_for("real", dtype, ref)
    worst = [0.0]

    def check(logits, rid, positions, what):
        got = logits.float().cpu()
        want = ref[rid][positions]
        err = float((got - want).abs().max())
        worst[0] = max(worst[0], err)
        assert err <= tol, f"{dtype} {what}: request {rid} positions {positions[0]}..{positions[-1]}: {err}"

    # whole prompt in one step (three 128-row tiles of the tensor-core attention in bfloat16)
    core.open("a")
    rows = [0, 1, 127, 128, 255, 256, 299]
    check(core.step([StepEntry("a", seqs["a"], rows)]), "a", rows, "whole")
    core.close("a")
    # portions of "a" beside the whole of "b", then both decode one token at a time (the last steps replay a graph)
    core.open("a"), core.open("b")
    lg = core.step([StepEntry("a", seqs["a"][:130], [129]), StepEntry("b", seqs["b"][:40], [39])])
    check(lg[:1], "a", [129], "portion")
    check(lg[1:], "b", [39], "beside")
    lg = core.step([StepEntry("a", seqs["a"][130:290], [0, 159]), StepEntry("b", seqs["b"][40:41], [0])])
    check(lg[:2], "a", [130, 289], "second portion")
    check(lg[2:], "b", [40], "decode beside a portion")
    for t in range(4):
        lg = core.step([StepEntry("a", [seqs["a"][290 + t]], [0]), StepEntry("b", [seqs["b"][41 + t]], [0])])
        check(lg[:1], "a", [290 + t], f"decode {t}")
        check(lg[1:], "b", [41 + t], f"decode {t}")
    record(f"real sizes {dtype}", worst[0], logits_std(ref))
    assert dtype == "float32" or core.runner.graph_replays > 0
    core.runner.check_device_errors()
    core.close("a"), core.close("b")
    assert core.cache.free_pages() == 48
