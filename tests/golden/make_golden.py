"""Makes tests/golden/tiny_reference_logits.safetensors: logits of the reference's own model
code (1483795887/qwen3_from_scratch, ``Qwen3`` on its ``base`` components, float32, CPU) for
one tiny random model and one token sequence.

    python tests/golden/make_golden.py <path to the reference's src/ folder>

The model folder is written by this repository's random-weights writer with the
configuration and seed below (stored in float32, so that both sides read identical values);
the file records the folder's hash so that a drift of the random generator shows up as a
clear failure in tests/test_plain_vs_reference.py, not as a numeric mismatch.
"""

import hashlib
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CONFIG = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=256, hidden_size=64, hidden_act="silu",
    num_hidden_layers=2, max_position_embeddings=128, num_key_value_heads=2, num_attention_heads=4,
    head_dim=16, intermediate_size=128, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True)
SEED = 0
TOKEN_SEED = 1
NUM_TOKENS = 31


def folder_hash(folder):
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def token_ids():
    g = torch.Generator().manual_seed(TOKEN_SEED)
    return torch.randint(0, CONFIG["vocab_size"], (NUM_TOKENS,), generator=g).tolist()


def write_folder(folder):
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    write_random_model(folder, config_from_dict(CONFIG), SEED, dtype="float32")


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path to the reference's src folder>")
    ref_src = sys.argv[1]
    sys.path.insert(0, ref_src)
    from qwen3_from_scratch.factory.config import load_from_file
    from qwen3_from_scratch.inference.context import ModelContext, set_forward_context
    from qwen3_from_scratch.models.parameter_loader import ParameterLoader
    from qwen3_from_scratch.models.qwen3 import Qwen3
    from safetensors.torch import save_file

    with tempfile.TemporaryDirectory() as folder:
        write_folder(folder)
        config = load_from_file(os.path.join(folder, "config.json"))
        loader = ParameterLoader()
        loader.load(folder)
        model = Qwen3(config)
        model.load_state(loader)
        model.eval()
        ids = token_ids()
        x = torch.tensor(ids).unsqueeze(0)
        ctx = ModelContext()
        ctx.dtype = torch.float32
        ctx.position_ids = torch.arange(0, x.shape[1]).unsqueeze(0)
        set_forward_context(ctx)
        with torch.no_grad():
            logits = model(x)[0].float().contiguous()
        meta = {"config": json.dumps(CONFIG), "seed": str(SEED), "token_seed": str(TOKEN_SEED),
                "folder_sha256": folder_hash(folder), "torch": torch.__version__,
                "source": "Qwen3.forward of the reference, base components, float32, CPU"}
        out = os.path.join(HERE, "tiny_reference_logits.safetensors")
        save_file({"logits": logits, "token_ids": torch.tensor(ids, dtype=torch.int32)}, out, metadata=meta)
        print("wrote", out, tuple(logits.shape), "max |logit|", float(logits.abs().max()))


if __name__ == "__main__":
    main()
