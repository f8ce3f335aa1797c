"""Makes tests/golden/tiny_*_reference_logits.safetensors: logits of the reference's own model
code (1483795887/qwen3_from_scratch, ``Qwen3`` on its ``base`` components, float32, CPU) for
two tiny random models and one token sequence each.

    python tests/golden/make_golden.py <path to the reference's src/ folder>

The two configurations differ in every size and option the reference reads: layers 2 / 3, width
64 / 80, heads 4:2 of 16 / 6:2 of 32 (heads x head size = / != width), feed-forward 128 / 200,
vocabulary 256 / 384, theta 1e4 / 1e6, eps 1e-6 / 1e-5, head tied / untied.  Each model folder is
written by this repository's random-weights writer with the configuration and seed below (stored
in float32, so that both sides read identical values); the file records the folder's hash so that
a drift of the random generator shows up as a clear failure in tests/test_plain_vs_reference.py,
not as a numeric mismatch.
"""

import hashlib
import json
import os
import sys
import tempfile

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CASES = {
    "tiny_reference_logits.safetensors": dict(
        config=dict(
            architectures=["Qwen3ForCausalLM"], vocab_size=256, hidden_size=64, hidden_act="silu",
            num_hidden_layers=2, max_position_embeddings=128, num_key_value_heads=2, num_attention_heads=4,
            head_dim=16, intermediate_size=128, rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True),
        seed=0, token_seed=1, num_tokens=31),
    "tiny_b_reference_logits.safetensors": dict(
        config=dict(
            architectures=["Qwen3ForCausalLM"], vocab_size=384, hidden_size=80, hidden_act="silu",
            num_hidden_layers=3, max_position_embeddings=256, num_key_value_heads=2, num_attention_heads=6,
            head_dim=32, intermediate_size=200, rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False),
        seed=2, token_seed=3, num_tokens=100),
}


def folder_hash(folder):
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        return hashlib.sha256(f.read()).hexdigest()


def token_ids(case):
    g = torch.Generator().manual_seed(case["token_seed"])
    return torch.randint(0, case["config"]["vocab_size"], (case["num_tokens"],), generator=g).tolist()


def write_folder(folder, case):
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    write_random_model(folder, config_from_dict(case["config"]), case["seed"], dtype="float32")


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

    for name, case in CASES.items():
        with tempfile.TemporaryDirectory() as folder:
            write_folder(folder, case)
            config = load_from_file(os.path.join(folder, "config.json"))
            loader = ParameterLoader()
            loader.load(folder)
            model = Qwen3(config)
            model.load_state(loader)
            model.eval()
            ids = token_ids(case)
            x = torch.tensor(ids).unsqueeze(0)
            ctx = ModelContext()
            ctx.dtype = torch.float32
            ctx.position_ids = torch.arange(0, x.shape[1]).unsqueeze(0)
            set_forward_context(ctx)
            with torch.no_grad():
                logits = model(x)[0].float().contiguous()
            meta = {"config": json.dumps(case["config"]), "seed": str(case["seed"]),
                    "token_seed": str(case["token_seed"]), "folder_sha256": folder_hash(folder),
                    "torch": torch.__version__,
                    "source": "Qwen3.forward of the reference, base components, float32, CPU"}
            out = os.path.join(HERE, name)
            save_file({"logits": logits, "token_ids": torch.tensor(ids, dtype=torch.int32)}, out, metadata=meta)
            print("wrote", out, tuple(logits.shape), "max |logit|", float(logits.abs().max()))


if __name__ == "__main__":
    main()
