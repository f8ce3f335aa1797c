"""Shared fixtures: tiny model folders with random weights, made in temporary folders."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
if os.path.dirname(os.path.abspath(__file__)) not in sys.path:
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA GPU here")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


# Tiny configurations of the architecture that differ in every size and option: layers, width,
# heads and group size, head size (B: heads * head_dim != width), feed-forward width (B: no
# multiple of 128), vocabulary, theta, eps, tied/untied head, positions, window.  A and B have
# full attention in every layer, like the reference's model, whose own logits for both are kept
# under tests/golden/; C, D and E have windowed layers.
TINY_A = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=256, hidden_size=64, hidden_act="silu",
    num_hidden_layers=2, max_position_embeddings=512, num_key_value_heads=2, num_attention_heads=4,
    head_dim=16, intermediate_size=128, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True)
TINY_B = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=384, hidden_size=80, hidden_act="silu",
    num_hidden_layers=3, max_position_embeddings=256, num_key_value_heads=2, num_attention_heads=6,
    head_dim=32, intermediate_size=200, rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False)
# the same with windowed layers, written the older way (use_sliding_window + max_window_layers)
TINY_E = dict(TINY_B, max_position_embeddings=1024, sliding_window=24, use_sliding_window=True, max_window_layers=1)
# a third one with a head size that is no power of two and one kv head
TINY_C = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=331, hidden_size=96, hidden_act="silu",
    num_hidden_layers=2, max_position_embeddings=768, num_key_value_heads=1, num_attention_heads=5,
    head_dim=48, intermediate_size=136, rms_norm_eps=1e-6, rope_theta=50000.0, tie_word_embeddings=False,
    layer_types=["sliding_attention", "full_attention"], sliding_window=40)

# and one with the head size the serving kernels are made for (128, pages of 16: the TMA decode kernel, the
# tcgen05 portion kernel and product, the decode step without norm and qkv_post kernels), heads * head_dim
# != width, a windowed layer beside a full one
TINY_D = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=500, hidden_size=256, hidden_act="silu",
    num_hidden_layers=2, max_position_embeddings=1024, num_key_value_heads=2, num_attention_heads=4,
    head_dim=128, intermediate_size=384, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True,
    layer_types=["full_attention", "sliding_attention"], sliding_window=100)

TINY = {"a": (TINY_A, 0), "b": (TINY_B, 2), "c": (TINY_C, 5), "d": (TINY_D, 9), "e": (TINY_E, 4)}


def make_folder(tmp_path_factory, key, dtype="bfloat16", float32_tensors=None):
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    config, seed = TINY[key]
    folder = str(tmp_path_factory.mktemp(f"tiny_{key}"))
    write_random_model(folder, config_from_dict(config), seed, dtype=dtype, float32_tensors=float32_tensors)
    return folder


@pytest.fixture(scope="session")
def tiny_folders(tmp_path_factory):
    """Model folders of the tiny configurations, weights stored in bfloat16."""
    return {key: make_folder(tmp_path_factory, key) for key in TINY}


def random_tokens(vocab_size, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab_size, (n,), generator=g).tolist()
