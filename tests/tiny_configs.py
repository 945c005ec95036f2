"""The tiny configurations the tests run: they differ in every size and option.

A: 2 layers, hidden 64, 4 query heads over 2 KV heads, head_dim 16, intermediate 128,
   vocabulary 256, theta 1e4, eps 1e-6, tied head, all keys in every layer.
B: 3 layers, hidden 96, 8 query heads over 2 KV heads, head_dim 32 (heads*head_dim !=
   hidden), intermediate 160, vocabulary 384, theta 1e6, eps 1e-5, untied head; layer 0
   sees all keys, layers 1 and 2 a window of 37 keys (no multiple of the page size).
B0 is B without the window (the shape the reference's own classes can run).
"""

import copy

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "tie_word_embeddings": True,
    "attention_bias": False, "hidden_act": "silu", "rope_scaling": None,
    "sliding_window": None, "use_sliding_window": False, "max_position_embeddings": 4096,
}

TINY_B0 = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3",
    "vocab_size": 384, "hidden_size": 96, "intermediate_size": 160, "num_hidden_layers": 3,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 32,
    "rms_norm_eps": 1e-5, "rope_theta": 1000000.0, "tie_word_embeddings": False,
    "attention_bias": False, "hidden_act": "silu", "rope_scaling": None,
    "sliding_window": None, "use_sliding_window": False, "max_position_embeddings": 4096,
}

TINY_B = copy.deepcopy(TINY_B0)
TINY_B.update({"sliding_window": 37, "use_sliding_window": True, "max_window_layers": 1})

CONFIGS = {"A": (TINY_A, 0), "B": (TINY_B, 1)}      # name -> (config.json content, seed)
ALL_CONFIGS = dict(CONFIGS, B0=(TINY_B0, 1))        # B0: what the reference's own classes can run


def make_folder(tmp_path, name):
    """Write the tiny model `name` with random weights into tmp_path/name; returns the folder."""
    from socrates_b200.config import config_from_dict
    from socrates_b200.weights import write_model_folder
    cfg_dict, seed = ALL_CONFIGS[name]
    return write_model_folder(config_from_dict(cfg_dict), seed, tmp_path / name)
