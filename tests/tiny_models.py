"""The tests' own small configurations and helpers to write them as model folders.

A and B are the two tiny Qwen3 configurations that differ in every size and option (heads and
groups, head size, sizes that are no power of two, layers, vocabulary, eps, theta, tying,
biases); C adds what A and B lack: no grouping (as many key/value heads as query heads), a
head size of 48, and a sliding window on two of its four layers.
"""
import json
import os

import torch

TINY_A = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "vocab_size": 256,
    "max_position_embeddings": 128, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "attention_bias": False, "hidden_act": "silu", "eos_token_id": 7,
}
TINY_B = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 96, "intermediate_size": 208, "num_hidden_layers": 3,
    "num_attention_heads": 6, "num_key_value_heads": 1, "head_dim": 32, "vocab_size": 311,
    "max_position_embeddings": 256, "rope_theta": 1000000.0, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": False, "attention_bias": True, "hidden_act": "silu", "eos_token_id": [5, 9],
}
TINY_C = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 80, "intermediate_size": 112, "num_hidden_layers": 4,
    "num_attention_heads": 5, "num_key_value_heads": 5, "head_dim": 48, "vocab_size": 199,
    "max_position_embeddings": 320, "rope_theta": 50000.0, "rms_norm_eps": 3e-6,
    "tie_word_embeddings": True, "attention_bias": False, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 24,
    "layer_types": ["full_attention", "sliding_attention", "full_attention", "sliding_attention"],
}
# D has the head size (64) and group size (4) that the bfloat16 attention kernels take, so that the
# engine tests run them and not only the plain kernels.
TINY_D = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 128, "intermediate_size": 320, "num_hidden_layers": 2,
    "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 64, "vocab_size": 500,
    "max_position_embeddings": 512, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": False, "attention_bias": False, "hidden_act": "silu",
}
# E has a head size of 128, which the tensor-memory attention kernel takes, and a window on one layer.
TINY_E = {
    "architectures": ["Qwen3ForCausalLM"], "hidden_size": 192, "intermediate_size": 256, "num_hidden_layers": 2,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128, "vocab_size": 389,
    "max_position_embeddings": 640, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6,
    "tie_word_embeddings": True, "attention_bias": False, "hidden_act": "silu",
    "use_sliding_window": True, "sliding_window": 150, "layer_types": ["full_attention", "sliding_attention"],
}
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


def write_model(folder, cfg_dict, seed, std=None):
    """A model folder with random weights (the library's random-weights mode).  ``std``
    rescales the matrices so that the layers matter more than at N(0, 0.02)."""
    from rocml_b200.config import config_from_dict
    from rocml_b200.weights import write_random_model

    cfg = config_from_dict(cfg_dict)
    write_random_model(folder, cfg, seed)
    if std is not None:
        from safetensors.torch import load_file, save_file
        path = os.path.join(folder, "model.safetensors")
        w = load_file(path)
        for k in w:
            if w[k].dim() == 2:
                w[k] = (w[k].float() * (std / 0.02)).to(torch.bfloat16)
        save_file(w, path)
    return folder


def prompt(seed, n, vocab):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
