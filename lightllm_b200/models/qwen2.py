"""``Qwen2ForCausalLM``: the dense decoder the reference runs (src/engine/engine_server.cpp).

Tensor names as the reference binds them (engine_server.cpp:436-450) plus the q/k/v biases and
``lm_head.weight``, which it never reads.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

from ..config import (ConfigError, ConfigReader, LayerSpec, ModelConfig, ModelSpec, PartSpec, RunEntry,
                      architecture_name, register_architecture)


@dataclass(frozen=True)
class Qwen2Config(ModelConfig):
    """Configuration of ``Qwen2ForCausalLM`` (dense decoder: GQA attention with QKV bias,
    NeoX rotary positions, RMSNorm, SwiGLU, optionally tied embeddings).

    Keys and fallbacks follow src/model/model_config.cpp:86-102 (``num_key_value_heads``
    defaults to ``num_attention_heads``, head size defaults to hidden/heads); the
    defaults of ``rms_norm_eps`` and ``rope_theta`` are the struct's
    (include/lightllm/model/model_config.h:20,23).  ``head_dim``, the window keys and
    ``tie_word_embeddings`` are honoured although the reference ignores them.
    """

    vocab_size: int = 0
    hidden_size: int = 0
    intermediate_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    rms_norm_eps: float = 1e-6
    rope_theta: float = 10000.0
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = False
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: int = 0
    hidden_act: str = "silu"

    @staticmethod
    def from_dict(raw: Dict[str, Any], where: str = "config.json") -> "Qwen2Config":
        r = ConfigReader(raw, where)
        arch = architecture_name(raw, where)
        hidden = r.integer("hidden_size")
        heads = r.integer("num_attention_heads")
        kv_heads = r.integer("num_key_value_heads", heads)
        head_dim = r.integer("head_dim", None)
        if head_dim is None:
            if hidden % heads != 0:
                raise ConfigError(
                    f"{where}: 'hidden_size' {hidden} is not a multiple of 'num_attention_heads' {heads} "
                    "and no 'head_dim' is given")
            head_dim = hidden // heads
        if heads % kv_heads != 0:
            raise ConfigError(
                f"{where}: 'num_attention_heads' {heads} is not a multiple of 'num_key_value_heads' {kv_heads}")
        if head_dim % 2 != 0:
            raise ConfigError(f"{where}: 'head_dim' {head_dim} must be even for rotary positions")
        act = r.string("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"{where}: 'hidden_act' must be 'silu' for {arch}, got {act!r}")
        if raw.get("rope_scaling") not in (None, {}):
            raise ConfigError(f"{where}: 'rope_scaling' is not supported for {arch}: {raw['rope_scaling']!r}")
        layers = r.integer("num_hidden_layers")
        use_window = r.boolean("use_sliding_window", False)
        window = r.integer("sliding_window", None)
        max_window_layers = r.integer("max_window_layers", layers, minimum=0)
        if use_window and window is None:
            raise ConfigError(f"{where}: 'use_sliding_window' is true but 'sliding_window' is missing")
        return Qwen2Config(
            architecture=arch,
            raw=dict(raw),
            vocab_size=r.integer("vocab_size"),
            hidden_size=hidden,
            intermediate_size=r.integer("intermediate_size"),
            num_hidden_layers=layers,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=r.real("rms_norm_eps", 1e-6),
            rope_theta=r.real("rope_theta", 10000.0),
            max_position_embeddings=r.integer("max_position_embeddings"),
            tie_word_embeddings=r.boolean("tie_word_embeddings", False),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=max_window_layers,
            hidden_act=act,
        )

    def layer_window(self, layer: int) -> Optional[int]:
        """Window of a layer's attention: the first ``max_window_layers`` layers see every
        earlier token; later ones see the last ``sliding_window`` tokens (self included)
        when ``use_sliding_window`` is set."""
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None



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
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": D}, head_prefix),
        # checkpoints written by other tools store the rotary frequencies, which are recomputed here
        ignored_suffixes=("rotary_emb.inv_freq",))


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_spec)
