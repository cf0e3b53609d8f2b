"""The tests' own small configurations. They differ in every size and option: head counts
and groups, head size, widths that are no power of two, layers, vocabulary, eps, rope rule,
tied or separate output matrix, window, page size, weight scale."""
import os

import torch

TINY_A = {  # 2 layers, 4 heads in 2 groups, head 16, tied, plain rope
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 64, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 128, "vocab_size": 256,
    "max_position_embeddings": 128, "rope_theta": 10000.0, "rope_scaling": None,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
}
TINY_B = {  # 3 layers, 3 heads on 1 kv head, head 32, hidden 96, untied, llama3 rope
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 96, "num_hidden_layers": 3, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 224, "vocab_size": 384,
    "max_position_embeddings": 256, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 32},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
}
TINY_C = {  # 4 layers, 6 heads in 3 groups, head 48 (hidden 80 != heads*head), windows on 2 layers
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 80, "num_hidden_layers": 4, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 176, "vocab_size": 200,
    "max_position_embeddings": 512, "rope_theta": 20000.0,
    "rope_scaling": {"rope_type": "linear", "factor": 2.0},
    "rms_norm_eps": 3e-6, "tie_word_embeddings": True, "sliding_window": 24,
    "layer_types": ["sliding_attention", "full_attention", "sliding_attention", "full_attention"],
}

TINY_D = {  # head size 64 (the tensor-core attention kernels), 6 heads in 2 groups, hidden 192, untied
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 192, "num_hidden_layers": 2, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 320, "vocab_size": 640,
    "max_position_embeddings": 1024, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False,
}
TINY_E = {  # head size 128, 4 heads on 1 kv head (group of 4), hidden 136 != heads * head, a window layer
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 136, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 128, "intermediate_size": 264, "vocab_size": 520,
    "max_position_embeddings": 1024, "rope_theta": 10000.0, "rope_scaling": None,
    "rms_norm_eps": 2e-6, "tie_word_embeddings": True, "sliding_window": 80,
    "layer_types": ["full_attention", "sliding_attention"],
}
TINY_F = {  # biases on q, k, v (drawn non-zero); full multi-head attention (4 kv heads), head 64, hidden 128
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 4,
    "num_key_value_heads": 4, "head_dim": 64, "intermediate_size": 288, "vocab_size": 300,
    "max_position_embeddings": 512, "rope_theta": 10000.0, "rope_scaling": None,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": False, "attention_bias": True,
}

# name -> (config, seed, weight std, norm std, page size)
TINY = {
    "A": (TINY_A, 0, 0.02, 0.0, 16),
    "B": (TINY_B, 1, 0.05, 0.1, 8),
    "C": (TINY_C, 2, 0.08, 0.2, 4),
    "D": (TINY_D, 3, 0.04, 0.1, 16),
    "E": (TINY_E, 4, 0.05, 0.0, 8),
    "F": (TINY_F, 5, 0.06, 0.1, 16),
}


def make_model_dir(root, name, dtype=torch.bfloat16):
    from rllm_b200.weights import write_random_model
    cfg, seed, std, norm_std, _ = TINY[name]
    d = os.path.join(str(root), f"tiny_{name}_{str(dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_random_model(cfg, seed, d, std=std, norm_std=norm_std, dtype=dtype)
    return d


def random_prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
