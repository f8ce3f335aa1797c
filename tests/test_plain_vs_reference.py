"""The plain implementation against the reference's own model code (golden logits made on the
CPU by tests/golden/make_golden.py from 1483795887/qwen3_from_scratch's ``Qwen3``)."""

import hashlib
import json
import os

import pytest
import torch
from safetensors import safe_open

import plain_qwen3 as plain

GOLDEN_DIR = os.path.join(os.path.dirname(__file__), "golden")


@pytest.mark.parametrize("name", ["tiny_reference_logits.safetensors", "tiny_b_reference_logits.safetensors"])
def test_plain_matches_reference_logits(tmp_path, name):
    """Tiny A (tied head, theta 1e4, eps 1e-6, 4:2 heads of 16) and tiny B (untied head, theta 1e6, eps 1e-5,
    6:2 heads of 32 on a width of 80, feed-forward of 200, three layers, 100 tokens)."""
    GOLDEN = os.path.join(GOLDEN_DIR, name)
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    with safe_open(GOLDEN, framework="pt") as f:
        meta = f.metadata()
        want = f.get_tensor("logits")
        ids = f.get_tensor("token_ids").tolist()
    config = json.loads(meta["config"])
    folder = str(tmp_path / "model")
    write_random_model(folder, config_from_dict(config), int(meta["seed"]), dtype="float32")
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()
    assert digest == meta["folder_sha256"], (
        "the random-weights writer no longer produces the folder the golden logits were made from; "
        "run tests/golden/make_golden.py again")
    cfg, weights = plain.read_model_folder(folder)
    got = plain.forward_logits(cfg, weights, ids)
    assert got.shape == want.shape
    # float32 on both sides, different order of operations: agreement to a few ulp of the logits' scale
    scale = float(want.abs().max())
    assert float((got - want).abs().max()) <= 2e-6 * max(scale, 1.0)


def test_plain_float64_agrees_with_float32(tmp_path):
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    from conftest import TINY_B, random_tokens
    folder = str(tmp_path / "model")
    write_random_model(folder, config_from_dict(TINY_B), 2)
    cfg, w32 = plain.read_model_folder(folder)
    _, w64 = plain.read_model_folder(folder, dtype=torch.float64)
    ids = random_tokens(cfg["vocab_size"], 70, 3)
    a = plain.forward_logits(cfg, w32, ids)
    b = plain.forward_logits(cfg, w64, ids)
    assert float((a.double() - b).abs().max()) < 1e-5
