"""Tiny configurations of Qwen2ForCausalLM for the tests.  A and B differ in every size and
option; C adds a window on its upper layers, so that it has two cache groups."""
import copy

TINY_A = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "intermediate_size": 172, "vocab_size": 512, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "use_sliding_window": False,
    "hidden_act": "silu",
}
TINY_B = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 1000, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 256, "use_sliding_window": False,
    "sliding_window": 4096, "max_window_layers": 3, "hidden_act": "silu",
}
TINY_C = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 3, "hidden_size": 80, "num_attention_heads": 5, "num_key_value_heads": 5,
    "head_dim": 48, "intermediate_size": 200, "vocab_size": 777, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 384, "use_sliding_window": True,
    "sliding_window": 20, "max_window_layers": 1, "hidden_act": "silu",
}
# D has heads of 64 (the tensor-core attention path in bfloat16), groups of 3 and a window on its last layer.
TINY_D = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 136, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 344, "vocab_size": 1537, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "max_position_embeddings": 1024, "use_sliding_window": True,
    "sliding_window": 150, "max_window_layers": 1, "hidden_act": "silu",
}
# E has heads of 128 (the head size of the larger checkpoints of the family), given by its own key since it is not
# hidden / heads, an untied head and no window.
TINY_E = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 128, "intermediate_size": 520, "vocab_size": 2003, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "use_sliding_window": False,
    "hidden_act": "silu",
}
PAGE_SIZE = {"A": 16, "B": 8, "C": 16, "D": 16, "E": 16}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def config(name):
    return copy.deepcopy(CONFIGS[name])
