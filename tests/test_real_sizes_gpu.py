"""Whole models at the layer sizes of Qwen3-0.6B, Qwen3-8B and Qwen3-32B (two layers each, the 0.6B one
with the full vocabulary of 151,936, the others with 4,999 entries) against the plain implementation,
in float32 and in bfloat16, under every way of cutting the work.  At these widths the kernels take other
branches than at the tiny configurations: the few-rows product splits its reduction and fetches ahead
differently, the tcgen05 product takes its 256-wide tiles, the decode attention cuts a context into
several ranges, and steps of 9 to 16 rows use the second token tile.

The folders are written here with the safetensors package from tensors drawn on the GPU (the engine's
own writer draws on the CPU, which would take a minute at these sizes); the plain implementation reads
the same files and runs in float64 on the GPU.
"""

import json
import os

import pytest
import torch

import plain_qwen3 as plain
from conftest import random_tokens
from harness import Replayer, assert_close

pytestmark = pytest.mark.gpu

PAGE = 16
SIZES = {
    "0.6b": dict(hidden_size=1024, num_attention_heads=16, num_key_value_heads=8, intermediate_size=3072,
                 vocab_size=151936, tie_word_embeddings=True),
    "8b": dict(hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, intermediate_size=12288,
               vocab_size=4999, tie_word_embeddings=False),
    "32b": dict(hidden_size=5120, num_attention_heads=64, num_key_value_heads=8, intermediate_size=25600,
                vocab_size=4999, tie_word_embeddings=False),
}
LONG = 330  # (and two of 800 and 1,024, run whole only)
SHORT = [24 + 2 * i for i in range(16)]  # sixteen short requests, 24 to 54 tokens


def config_of(size):
    return dict(architectures=["Qwen3ForCausalLM"], hidden_act="silu", num_hidden_layers=2,
                max_position_embeddings=4096, head_dim=128, rms_norm_eps=1e-6, rope_theta=1000000.0, **SIZES[size])


def write_folder(folder, cfg, seed):
    """config.json + model.safetensors under the checkpoint's tensor names, bfloat16: matrices N(0, 0.02),
    norm weights 1 + N(0, 0.1)."""
    from safetensors.torch import save_file
    g = torch.Generator(device="cuda").manual_seed(seed)
    H, D, I, V = cfg["hidden_size"], cfg["head_dim"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv = cfg["num_attention_heads"], cfg["num_key_value_heads"]

    def matrix(*shape):
        return (torch.randn(*shape, generator=g, device="cuda") * 0.02).to(torch.bfloat16).cpu()

    def vector(n):
        return (1 + 0.1 * torch.randn(n, generator=g, device="cuda")).to(torch.bfloat16).cpu()

    t = {"model.embed_tokens.weight": matrix(V, H), "model.norm.weight": vector(H)}
    if not cfg["tie_word_embeddings"]:
        t["lm_head.weight"] = matrix(V, H)
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}"
        t[f"{p}.input_layernorm.weight"] = vector(H)
        t[f"{p}.post_attention_layernorm.weight"] = vector(H)
        t[f"{p}.self_attn.q_proj.weight"] = matrix(hq * D, H)
        t[f"{p}.self_attn.k_proj.weight"] = matrix(hkv * D, H)
        t[f"{p}.self_attn.v_proj.weight"] = matrix(hkv * D, H)
        t[f"{p}.self_attn.o_proj.weight"] = matrix(H, hq * D)
        t[f"{p}.self_attn.q_norm.weight"] = vector(D)
        t[f"{p}.self_attn.k_norm.weight"] = vector(D)
        t[f"{p}.mlp.gate_proj.weight"] = matrix(I, H)
        t[f"{p}.mlp.up_proj.weight"] = matrix(I, H)
        t[f"{p}.mlp.down_proj.weight"] = matrix(H, I)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file(t, os.path.join(folder, "model.safetensors"))


def sequences(size):
    vocab = SIZES[size]["vocab_size"]
    seqs = {"long": random_tokens(vocab, LONG, 500)}
    for i, n in enumerate(SHORT):
        seqs[f"s{i}"] = random_tokens(vocab, n, 600 + i)
    seqs["late"] = random_tokens(vocab, 70, 700)
    # enough rows for the products that have the work of the kernel after them in their epilogue (QKV with head norm,
    # rotation and page write; gate/up with SwiGLU): by single CTAs at 800 rows, by pairs of CTAs at 1,024
    seqs["longer"] = random_tokens(vocab, 800, 800)
    seqs["longest"] = random_tokens(vocab, 1024, 801)
    return seqs


@pytest.fixture(scope="module", params=list(SIZES))
def model(request, tmp_path_factory):
    """(size, folder, sequences, plain logits of every position of every sequence)."""
    size = request.param
    folder = str(tmp_path_factory.mktemp(f"real_{size.replace('.', '_')}"))
    cfg = config_of(size)
    write_folder(folder, cfg, seed=11)
    seqs = sequences(size)
    _, w = plain.read_model_folder(folder, dtype=torch.float64)
    w = {k: v.cuda() for k, v in w.items()}
    with torch.no_grad():
        want = {r: plain.forward_logits(cfg, w, ids).float().cpu() for r, ids in seqs.items()}
    del w
    torch.cuda.empty_cache()
    return size, folder, seqs, want


def make_session(folder, dtype, cache_tokens, **kw):
    from qwen3_from_scratch_b200.engine.session import Session
    return Session(folder, dtype=dtype, page_size=PAGE, cache_tokens=cache_tokens, max_seqs=24, max_step_tokens=1024,
                   **kw)


def subset(d, keys):
    return {k: d[k] for k in keys}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_decoded_and_in_portions(model, dtype):
    size, folder, seqs, want = model
    session = make_session(folder, dtype, cache_tokens=4096)
    # each request alone and whole
    rep = Replayer(session, seqs)
    for req, ids in seqs.items():
        rep.step([(req, len(ids))])
    assert_close(rep.result(), want, dtype, f"{size} whole")
    # most of it in one step, the last 32 tokens one by one (a batch of one row)
    some = subset(seqs, ["long", "s3", "s15"])
    rep = Replayer(session, some)
    for req, ids in some.items():
        head = max(0, len(ids) - 32)
        if head:
            rep.step([(req, head)])
        while rep.remaining(req):
            rep.step([(req, 1)])
    assert_close(rep.result(), subset(want, some), dtype, f"{size} prefix + 32 single tokens")
    # portions of changing size, down to two tokens
    some = subset(seqs, ["long", "s8"])
    rep = Replayer(session, some)
    sizes = [16, 7, 5, 3, 2, 2, 130, 11, 1, 2, 29]
    for req in some:
        i = 0
        while rep.remaining(req):
            rep.step([(req, sizes[i % len(sizes)])])
            i += 1
    assert_close(rep.result(), subset(want, some), dtype, f"{size} portions")
    session.manager.check()
    assert not session.manager.live_requests()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_with_page_reuse(model, dtype):
    """Up to four live requests, a portion of the long one beside single tokens of others, in a pool that
    holds the long request and little more, so that the short ones' pages are used again and again."""
    size, folder, seqs, want = model
    some = subset(seqs, ["long", "s0", "s5", "s9", "s12", "s14", "s2"])
    pages_of = {r: -(-len(ids) // PAGE) for r, ids in some.items()}
    total_pages = pages_of["long"] + 2 * max(pages_of[r] for r in some if r != "long") + 1
    session = make_session(folder, dtype, cache_tokens=total_pages * PAGE, poison_freed_pages=True)
    rep = Replayer(session, some)
    waiting, live = list(some), []
    portion = [13, 2, 40, 1, 9, 3]
    tick = 0
    while waiting or live:
        while waiting and len(live) < 4 and sum(pages_of[r] for r in live) + pages_of[waiting[0]] <= total_pages:
            live.append(waiting.pop(0))
        assert live
        step = []
        for j, req in enumerate(live):
            # requests past their first portion decode token by token, except the oldest, which brings portions
            n = portion[(tick + j) % len(portion)] if (j == 0 or rep.fed[req] == 0) else 1
            step.append((req, n))
        rep.step(step)
        session.manager.check()
        live = [r for r in live if rep.remaining(r)]
        tick += 1
    assert not session.manager.live_requests()
    assert_close(rep.result(), subset(want, some), dtype, f"{size} mixed")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sixteen_twelve_and_eight_rows_decoding_together(model, dtype):
    """Sixteen requests decode together for three steps, twelve for two more, eight for three more; in the
    second step a prompt portion of another request arrives beside the sixteen single tokens."""
    size, folder, seqs, want = model
    some = subset(seqs, [f"s{i}" for i in range(16)] + ["late"])
    session = make_session(folder, dtype, cache_tokens=2048)
    rep = Replayer(session, some)
    left = {f"s{i}": (8 if i < 8 else 5 if i < 12 else 3) for i in range(16)}
    for req, n in left.items():
        rep.step([(req, len(some[req]) - n)], end_finished=False)
    for step in range(8):
        rows = [(req, 1) for req in left if rep.remaining(req)]
        assert len(rows) == (16 if step < 3 else 12 if step < 5 else 8)
        if step == 1:
            rows.insert(5, ("late", 40))
        rep.step(rows)
    rep.step([("late", 30)])
    assert not session.manager.live_requests()
    assert_close(rep.result(), subset(want, some), dtype, f"{size} decode batches")
