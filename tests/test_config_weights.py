"""Configuration, registry, safetensors reading and the loader's one clear error (no GPU)."""
import json
import os

import pytest
import torch

from lightllm_b200.models.qwen2 import Qwen2Config
from lightllm_b200.config import (ConfigError, config_from_dict, known_architectures, load_config,
                                  model_spec_for)
from lightllm_b200.models import Model, weight_specs_of
from lightllm_b200.weights import (Checkpoint, SafetensorsError, WeightError, check_against, load_checkpoint_tensors,
                                   random_tensors, save_file, write_random_model)
from tests.plain.qwen2_plain import read_safetensors
from tests.tiny_configs import config


def test_registry_knows_qwen2_and_rejects_others():
    assert "Qwen2ForCausalLM" in known_architectures()
    cfg = config("A")
    cfg["architectures"] = ["LlamaForCausalLM"]
    with pytest.raises(ConfigError, match="unknown architecture 'LlamaForCausalLM'.*Qwen2ForCausalLM"):
        config_from_dict(cfg)
    with pytest.raises(ConfigError, match="architectures"):
        config_from_dict({"hidden_size": 8})


def test_typed_config_defaults_and_derived_sizes():
    a = config_from_dict(config("A"))
    assert isinstance(a, Qwen2Config)
    assert (a.head_dim, a.num_key_value_heads, a.rms_norm_eps, a.rope_theta) == (16, 2, 1e-6, 10000.0)
    assert a.tie_word_embeddings and a.layer_window(1) is None
    b = config_from_dict(config("B"))
    assert (b.head_dim, b.num_key_value_heads, b.rms_norm_eps, b.rope_theta) == (32, 1, 1e-5, 1e6)
    minimal = {k: v for k, v in config("A").items() if k not in ("rms_norm_eps", "rope_theta", "num_key_value_heads")}
    m = config_from_dict(minimal)
    # absent keys take the struct's defaults, not 0 as in the reference's parser
    assert m.rms_norm_eps == 1e-6 and m.rope_theta == 10000.0 and m.num_key_value_heads == m.num_attention_heads
    c = config_from_dict(config("C"))
    assert [c.layer_window(i) for i in range(3)] == [None, 20, 20]


@pytest.mark.parametrize("key,value,match", [
    ("hidden_size", None, "required key 'hidden_size'"), ("vocab_size", 0, "'vocab_size' must be >= 1"),
    ("num_key_value_heads", 3, "not a multiple"), ("hidden_act", "gelu", "hidden_act"),
    ("rms_norm_eps", "x", "must be a number"), ("tie_word_embeddings", 1, "true or false"),
    ("rope_scaling", {"type": "yarn"}, "rope_scaling"), ("num_hidden_layers", 2.5, "must be an integer")])
def test_config_errors_name_the_key(key, value, match):
    cfg = config("A")
    if value is None:
        del cfg[key]
    else:
        cfg[key] = value
    with pytest.raises(ConfigError, match=match):
        config_from_dict(cfg)


def test_window_needs_its_size():
    cfg = config("C")
    del cfg["sliding_window"]
    with pytest.raises(ConfigError, match="sliding_window"):
        config_from_dict(cfg)


def test_spec_is_data_and_names_follow_the_checkpoint():
    spec = model_spec_for(config_from_dict(config("B")))
    assert len(spec.layers) == 3 and [e.layer for e in spec.run] == [0, 1, 2]
    names = {s.name: s.shape for s in weight_specs_of(spec)}
    assert names["model.layers.2.self_attn.k_proj.bias"] == (32,)
    assert names["model.layers.0.mlp.gate_proj.weight"] == (256, 96)
    assert names["lm_head.weight"] == (1000, 96)
    tied = {s.name for s in weight_specs_of(model_spec_for(config_from_dict(config("A"))))}
    assert "lm_head.weight" not in tied and "model.embed_tokens.weight" in tied
    c = Model(model_spec_for(config_from_dict(config("C"))))
    assert len(c.cache_layout.groups) == 2 and c.cache_layout.planes_per_group == [1, 2]


def test_random_model_roundtrip_and_seed(tmp_path):
    d1, d2, d3 = (str(tmp_path / n) for n in "abc")
    write_random_model(config("A"), 5, d1, "bfloat16")
    write_random_model(config("A"), 5, d2, "bfloat16")
    write_random_model(config("A"), 6, d3, "float32")
    assert load_config(d1).hidden_size == 64
    a, b, c = (read_safetensors(os.path.join(d, "model.safetensors")) for d in (d1, d2, d3))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    assert not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    w = c["model.layers.0.mlp.up_proj.weight"]
    assert abs(float(w.std()) - 0.02) < 0.002 and abs(float(c["model.norm.weight"].mean()) - 1.0) < 0.01
    ck = Checkpoint(d1)
    assert ck.tensors["model.norm.weight"].dtype == "BF16" and torch.equal(ck.read("model.norm.weight").float(), a["model.norm.weight"])
    ck.close()


def test_precision_policy(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    specs = weight_specs_of(model_spec_for(config_from_dict(config("A"))))
    t = random_tensors(specs, 1, torch.bfloat16)
    t["model.norm.weight"] = t["model.norm.weight"].float()          # one tensor stored in 32 bits
    save_file(t, os.path.join(d, "model.safetensors"))
    cpu = torch.device("cpu")
    got = load_checkpoint_tensors(d, specs, torch.bfloat16, cpu)
    assert got["model.norm.weight"].dtype == torch.float32            # stays 32-bit
    assert got["model.embed_tokens.weight"].dtype == torch.bfloat16
    got32 = load_checkpoint_tensors(d, specs, torch.float32, cpu)
    assert all(v.dtype == torch.float32 for v in got32.values())


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    d = str(tmp_path / "m")
    os.makedirs(d)
    specs = weight_specs_of(model_spec_for(config_from_dict(config("B"))))
    t = random_tensors(specs, 1, torch.float32)
    del t["model.layers.1.self_attn.q_proj.bias"]
    del t["lm_head.weight"]
    t["model.layers.9.extra.weight"] = torch.zeros(3)
    t["model.norm.weight"] = torch.zeros(95)
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(256, 96)
    save_file(t, os.path.join(d, "model.safetensors"))
    with pytest.raises(WeightError) as ei:
        load_checkpoint_tensors(d, specs, torch.float32, torch.device("cpu"))
    e = ei.value
    assert e.missing == ["lm_head.weight", "model.layers.1.self_attn.q_proj.bias"]
    assert e.unexpected == ["model.layers.9.extra.weight"]
    assert {n for n, _, _ in e.wrong_shape} == {"model.norm.weight", "model.layers.0.mlp.down_proj.weight"}
    msg = str(e)
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes (2)", "file has [95], model expects [96]"):
        assert needle in msg


def test_safetensors_errors(tmp_path):
    p = str(tmp_path / "x.safetensors")
    with pytest.raises(SafetensorsError, match="cannot open"):
        Checkpoint(str(tmp_path))
    open(p, "wb").write(b"\x05\x00")
    from lightllm_b200.weights import SafetensorsFile
    with pytest.raises(SafetensorsError, match="invalid safetensors header"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "F8_E4M3", "shape": [1], "data_offsets": [0, 1]}}).encode()
    open(p, "wb").write(len(hdr).to_bytes(8, "little") + hdr + b"\0")
    with pytest.raises(SafetensorsError, match="unknown safetensors dtype"):
        SafetensorsFile(p)
    hdr = json.dumps({"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 4]}}).encode()
    open(p, "wb").write(len(hdr).to_bytes(8, "little") + hdr + b"\0" * 4)
    with pytest.raises(SafetensorsError, match="byte size mismatch"):
        SafetensorsFile(p)
    save_file({"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "i": torch.arange(4, dtype=torch.int32)}, p)
    f = SafetensorsFile(p)
    assert torch.equal(f.read("a"), torch.arange(6, dtype=torch.float32).reshape(2, 3))
    with pytest.raises(SafetensorsError, match="tensor not found: nope"):
        f.read("nope")
    f.close()


def test_a_layer_is_a_list_of_sub_blocks():
    from lightllm_b200.config import LayerSpec, PartSpec, SubBlock
    n, m, f = PartSpec("rmsnorm"), PartSpec("attention"), PartSpec("gated_mlp")
    short = LayerSpec(n, m, n, f, arrangement="pre_norm")
    assert short.arrangement == "sequential" and [sb.role for sb in short.sub_blocks] == ["mixer", "ffn"]
    assert short.sub_blocks[0].norm_before is n and short.sub_blocks[1].norm_after is None
    lone = LayerSpec(sub_blocks=[SubBlock("mixer", m)])
    assert len(lone.sub_blocks) == 1 and lone.sub_blocks[0].norm_before is None
    with pytest.raises(ValueError, match="at most one mixer"):
        LayerSpec(sub_blocks=[SubBlock("mixer", m), SubBlock("mixer", m)])
    with pytest.raises(ValueError, match="at least one"):
        LayerSpec()
    with pytest.raises(ValueError, match="not both"):
        LayerSpec(n, m, sub_blocks=[SubBlock("ffn", f)])
    with pytest.raises(ValueError, match="role"):
        LayerSpec(sub_blocks=[SubBlock("norm", n)])
    with pytest.raises(ValueError, match="parallel"):
        LayerSpec(sub_blocks=[SubBlock("ffn", f, n, n, after="stream")], arrangement="parallel")
    with pytest.raises(ValueError, match="arrangement"):
        LayerSpec(n, m, n, f, arrangement="sandwich")


def test_end_of_sequence_ids_come_from_the_configuration():
    base = config("A")
    assert config_from_dict(base).eos_token_ids == ()
    assert config_from_dict({**base, "eos_token_id": 7}).eos_token_ids == (7,)
    assert config_from_dict({**base, "eos_token_id": [7, 9]}).eos_token_ids == (7, 9)
    with pytest.raises(ConfigError, match="eos_token_id"):
        config_from_dict({**base, "eos_token_id": "end"}).eos_token_ids
