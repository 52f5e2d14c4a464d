"""Shared fixtures: the two tiny Llama configurations and model folders made from them."""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu)")


# Two configurations that differ in every size and option: layers, width, heads,
# groups, head size, feed-forward width, vocabulary, theta, scaling, eps, tying.
TINY_A = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 160, "vocab_size": 256,
    "rope_theta": 10000.0, "rope_scaling": None, "rms_norm_eps": 1e-5,
    "tie_word_embeddings": True, "max_position_embeddings": 128, "torch_dtype": "bfloat16",
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3,
    "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 256, "vocab_size": 512,
    "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 256,
    "torch_dtype": "bfloat16", "eos_token_id": 7, "bos_token_id": 1,
}
# A third shape with sizes that are no power of two and a head size of 48.
TINY_C = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 120, "num_attention_heads": 6,
    "num_key_value_heads": 3, "head_dim": 48, "intermediate_size": 200, "vocab_size": 331,
    "rope_theta": 25000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 2.0, "original_max_position_embeddings": 32},
    "rms_norm_eps": 3e-6, "tie_word_embeddings": True, "max_position_embeddings": 512,
    "torch_dtype": "float32",
}
# A fourth with the head size (128) and lengths that the tcgen05 attention and the paired
# tcgen05 product take, so that the engine meets them and not only the kernel tests.
TINY_D = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 256, "num_attention_heads": 4,
    "num_key_value_heads": 2, "head_dim": 128, "intermediate_size": 384, "vocab_size": 300,
    "rope_theta": 100000.0, "rope_scaling": None, "rms_norm_eps": 2e-5,
    "tie_word_embeddings": False, "max_position_embeddings": 1024, "torch_dtype": "bfloat16",
}
# A fifth with heads of 64 in groups of three: the other head size that the tcgen05 attention
# and the TMA-fed decode attention take.
TINY_E = {
    "architectures": ["LlamaForCausalLM"],
    "num_hidden_layers": 2, "hidden_size": 192, "num_attention_heads": 6,
    "num_key_value_heads": 2, "head_dim": 64, "intermediate_size": 320, "vocab_size": 411,
    "rope_theta": 300000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 1024,
    "torch_dtype": "bfloat16",
}
TINY = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}


@pytest.fixture(scope="session")
def model_folders(tmp_path_factory):
    """name -> model folder with random weights (made once per test session)."""
    from simple_inference_b200.weights import write_random_model
    out = {}
    for i, (name, cfg) in enumerate(TINY.items()):
        out[name] = write_random_model(tmp_path_factory.mktemp(f"tiny_{name}"), cfg, seed=11 + i)
    return out


def random_ids(n: int, vocab: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
