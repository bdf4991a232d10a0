"""``Qwen2ForCausalLM``: the dense decoder the reference runs (src/engine/engine_server.cpp).

Tensor names as the reference binds them (engine_server.cpp:436-450) plus the q/k/v biases and
``lm_head.weight``, which it never reads.
"""
from __future__ import annotations

from ..config import LayerSpec, ModelSpec, PartSpec, Qwen2Config, RunEntry, register_architecture


def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    D = cfg.hidden_size
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}"
        layers.append(LayerSpec(
            norm1=PartSpec("rmsnorm", {"hidden_size": D, "eps": cfg.rms_norm_eps}, f"{p}.input_layernorm"),
            mixer=PartSpec("attention", {
                "hidden_size": D, "num_heads": cfg.num_attention_heads, "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim, "qkv_bias": True, "out_bias": False, "window": cfg.layer_window(i),
                "position": PartSpec("rotary", {"head_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                                "rotary_dim": cfg.head_dim, "style": "neox"}),
            }, f"{p}.self_attn"),
            norm2=PartSpec("rmsnorm", {"hidden_size": D, "eps": cfg.rms_norm_eps}, f"{p}.post_attention_layernorm"),
            ffn=PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": cfg.intermediate_size,
                                       "activation": cfg.hidden_act}, f"{p}.mlp"),
            arrangement="pre_norm"))
    head_prefix = "model.embed_tokens" if cfg.tie_word_embeddings else "lm_head"
    return ModelSpec(
        architecture=cfg.architecture, hidden_size=D, vocab_size=cfg.vocab_size,
        max_positions=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": D}, "model.embed_tokens"),
        layers=layers,
        run=[RunEntry(i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"hidden_size": D, "eps": cfg.rms_norm_eps}, "model.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": D}, head_prefix))


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_spec)
