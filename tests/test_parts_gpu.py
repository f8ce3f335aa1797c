"""Each part alone against its plain function, built with sizes of its own (no model around it),
and toy parts registered from here and run through the engine without a change to its files: a
mixer with state of its own, a feed-forward that routes tokens to experts, a position encoding the
fused kernel does not know; each in a toy architecture with its own configuration class."""

import json
import os
from dataclasses import dataclass

import pytest
import torch

import plain_qwen3 as plain
from harness import Replayer

pytestmark = pytest.mark.gpu

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def runtime(dtype, max_tokens=256, max_seqs=4):
    from qwen3_from_scratch_b200.parts.base import Runtime
    return Runtime(torch.device("cuda:0"), DT[dtype], max_tokens, max_seqs)


def random_weights(part, dtype, seed=0):
    """Random tensors for a part's specs: (device dict as the loader would give it, float64 CPU copies)."""
    g = torch.Generator().manual_seed(seed)
    dev, ref = {}, {}
    for s in part.weight_specs():
        if s.init == "one_plus_normal":
            t = 1 + 0.1 * torch.randn(s.shape, generator=g)
        else:
            t = 0.05 * torch.randn(s.shape, generator=g)
        stored = t.to(torch.float32 if s.kind == "vector" else DT[dtype])
        dev[s.name] = stored.cuda()
        ref[s.name] = stored.double()
    return dev, ref


def close(got, want, dtype):
    got, want = got.double().cpu(), want.double()
    err = float((got - want).abs().max()) / max(float(want.abs().max()), 1e-9)
    assert err <= TOL[dtype], f"relative error {err:.3g} > {TOL[dtype]:g}"


@pytest.mark.parametrize("dtype", list(DT))
def test_norm_part(dtype):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    part = create_part("norm", PartSpec("rms_norm", {"dim": 72, "eps": 1e-5}), name="n")
    dev, ref = random_weights(part, dtype)
    part.setup(runtime(dtype), dev)
    g = torch.Generator().manual_seed(1)
    stream = torch.randn(9, 72, generator=g)
    delta = torch.randn(9, 72, generator=g).to(DT[dtype])
    s = stream.cuda()
    out = part.add_norm(s, delta.cuda())
    close(s, stream.double() + delta.double(), "float32")
    close(out, plain.rms_norm(stream.double() + delta.double(), ref["n.weight"], 1e-5), dtype)
    x = torch.randn(5, 3, 72, generator=g).to(DT[dtype])
    close(part.forward(x.cuda()), plain.rms_norm(x.double(), ref["n.weight"], 1e-5), dtype)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("head_dim,rotary_dim", [(48, None), (64, 32)])
def test_position_part(dtype, head_dim, rotary_dim):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    part = create_part("position", PartSpec("rotary_neox", {"head_dim": head_dim, "theta": 12345.0,
                                                            "max_positions": 5000, "rotary_dim": rotary_dim}))
    part.setup(runtime(dtype), {})
    g = torch.Generator().manual_seed(2)
    x = torch.randn(20, 3, head_dim, generator=g).to(DT[dtype])
    positions = torch.tensor([0, 1, 2, 3, 4, 100, 101, 999, 4000, 4999, 7, 7, 7, 50, 51, 52, 53, 54, 55, 56],
                             dtype=torch.int32)
    out = part.apply(x.cuda(), positions.cuda())
    rot = rotary_dim or head_dim
    cos, sin = plain.rope_cos_sin(positions, rot, 12345.0, dtype=torch.float64)
    want = x.double().clone()
    want[..., :rot] = plain.apply_rope(x.double()[..., :rot], cos, sin)
    # the angle is a float32 product of position and frequency on both sides; sin/cos of an angle
    # of thousands of radians carry its rounding (2^-24 * 5000 ~ 3e-4) into the result
    tol = dict(TOL)
    tol["float32"] = 5e-4
    err = float((out.double().cpu() - want).abs().max()) / float(want.abs().max())
    assert err <= tol[dtype], err


@pytest.mark.parametrize("dtype", list(DT))
def test_feed_forward_part(dtype):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    part = create_part("feed_forward", PartSpec("swiglu", {"hidden_size": 56, "intermediate_size": 136}), name="f")
    dev, ref = random_weights(part, dtype)
    part.setup(runtime(dtype), dev)
    x = (torch.randn(13, 56, generator=torch.Generator().manual_seed(3)) * 2).to(DT[dtype])
    close(part.forward(x.cuda()), plain.swiglu_mlp(x.double(), ref, "f"), dtype)


@pytest.mark.parametrize("dtype", list(DT))
def test_embedding_and_head_parts(dtype):
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    emb = create_part("embedding", PartSpec("token_embedding", {"vocab_size": 211, "hidden_size": 40}), name="e")
    head = create_part("head", PartSpec("lm_head", {"vocab_size": 211, "hidden_size": 40, "tied_to": "e.weight"}),
                       name="h")
    assert head.weight_specs() == []
    dev, ref = random_weights(emb, dtype)
    rt = runtime(dtype)
    emb.setup(rt, dev)
    head.setup(rt, dev)
    ids = torch.tensor([0, 210, 5, 5, 17], dtype=torch.int32)
    stream = emb.forward(ids.cuda())
    assert stream.dtype == torch.float32
    close(stream, ref["e.weight"][ids.long()], "float32")
    x = torch.randn(4, 40, generator=torch.Generator().manual_seed(4)).to(DT[dtype])
    logits = head.forward(x.cuda())
    assert logits.dtype == torch.float32
    close(logits, x.double() @ ref["e.weight"].t(), dtype)


def mixer_context(part, rt, page_size, entries):
    """A cache manager, storage and batch for one mixer alone (cache id 0)."""
    from qwen3_from_scratch_b200.cache import CacheManager, layout_of
    from qwen3_from_scratch_b200.cache.storage import CacheStorage
    from qwen3_from_scratch_b200.engine.batch import BatchContext
    layout = layout_of({0: part.cache_spec()})
    manager = CacheManager(layout, page_size, 64, rt.max_seqs)
    storage = CacheStorage(layout, page_size, rt.max_seqs, rt.device, rt.dtype)
    return manager, storage, lambda: BatchContext(manager, storage, rt)


@pytest.mark.parametrize("dtype", list(DT))
@pytest.mark.parametrize("window", [None, 9])
def test_attention_part_whole_then_in_portions(dtype, window):
    from qwen3_from_scratch_b200.engine.batch import Entry
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    H, hq, hkv, d, eps, theta = 72, 6, 2, 48, 1e-5, 50000.0
    spec = PartSpec("gqa_attention", {
        "hidden_size": H, "num_heads": hq, "num_kv_heads": hkv, "head_dim": d, "qk_norm_eps": eps,
        "window": window,
        "position": PartSpec("rotary_neox", {"head_dim": d, "theta": theta, "max_positions": 4096})})
    part = create_part("mixer", spec, name="a")
    dev, ref = random_weights(part, dtype)
    rt = runtime(dtype)
    part.setup(rt, dev)
    n = 45
    x = torch.randn(n, H, generator=torch.Generator().manual_seed(5)).to(DT[dtype])
    cfg = {"head_dim": d, "rms_norm_eps": eps, "rope_theta": theta}
    want = plain.self_attention(x.double(), ref, "a", cfg, torch.arange(n), window)
    manager, storage, new_ctx = mixer_context(part, rt, 8, None)
    for cuts in ([n], [16, 1, 1, 7, 2, 18]):
        manager.open("r")
        got, at = [], 0
        for c in cuts:
            manager.reserve("r", at + c)
            ctx = new_ctx().build([Entry("r", [0] * c)], vocab_size=1)
            got.append(part.forward(x[at:at + c].cuda().contiguous(), ctx, 0, True).clone())
            at += c
            manager.advance("r", at)
        manager.close("r")
        close(torch.cat(got), want, dtype)
    assert int(rt.status.item()) == 0


@pytest.mark.parametrize("dtype", list(DT))
def test_block_part(dtype):
    from qwen3_from_scratch_b200.engine.batch import Entry
    from qwen3_from_scratch_b200.parts.base import PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    H, hq, hkv, d, inter, eps, theta = 48, 3, 1, 32, 100, 1e-6, 10000.0
    norm = PartSpec("rms_norm", {"dim": H, "eps": eps})
    block = create_part("block", PartSpec("pre_norm", {
        "norm1": norm, "norm2": norm,
        "mixer": PartSpec("gqa_attention", {
            "hidden_size": H, "num_heads": hq, "num_kv_heads": hkv, "head_dim": d, "qk_norm_eps": eps,
            "position": PartSpec("rotary_neox", {"head_dim": d, "theta": theta, "max_positions": 512})}),
        "feed_forward": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": inter}),
        "names": {"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm",
                  "feed_forward": "mlp"}}), name="model.layers.0")
    dev, ref = random_weights(block, dtype)
    rt = runtime(dtype)
    block.setup(rt, dev)
    n = 23
    x = torch.randn(n, H, generator=torch.Generator().manual_seed(6))
    cfg = {"head_dim": d, "rms_norm_eps": eps, "rope_theta": theta}
    want = plain.decoder_layer(x.double(), ref, 0, cfg, torch.arange(n), None)
    manager, storage, new_ctx = mixer_context(block.mixer, rt, 4, None)
    manager.open("r")
    manager.reserve("r", n)
    ctx = new_ctx().build([Entry("r", [0] * n)], vocab_size=1)
    stream = x.cuda()
    pending = block.forward(stream, None, ctx, 0, True)
    close(stream + pending.float(), want, dtype)


def test_block_part_few_rows_run_without_norm_kernels(monkeypatch):
    """Up to 16 rows in bfloat16: the block's output projections add into the stream themselves and leave its
    rows' sums of squares and the rows times the next norm's weight; the input projections run on that operand
    and apply 1 / rms (passed from one block to the next through the step's shared data).  Two calls of the
    block on caches of their own, as two layers with the same weights would be, against the plain layer
    applied twice; how many norm kernels run; and the same block made to take the path with norm kernels."""
    from qwen3_from_scratch_b200.cache import CacheManager, layout_of
    from qwen3_from_scratch_b200.cache.storage import CacheStorage
    from qwen3_from_scratch_b200.engine.batch import BatchContext, Entry
    from qwen3_from_scratch_b200.kernels import ops
    from qwen3_from_scratch_b200.parts.base import STREAM_SUMSQ, PartSpec
    from qwen3_from_scratch_b200.registry import create_part
    dtype = "bfloat16"
    H, hq, hkv, d, inter, eps, theta = 80, 4, 2, 32, 104, 1e-5, 10000.0
    norm = PartSpec("rms_norm", {"dim": H, "eps": eps})
    block = create_part("block", PartSpec("pre_norm", {
        "norm1": norm, "norm2": norm,
        "mixer": PartSpec("gqa_attention", {
            "hidden_size": H, "num_heads": hq, "num_kv_heads": hkv, "head_dim": d, "qk_norm_eps": eps,
            "position": PartSpec("rotary_neox", {"head_dim": d, "theta": theta, "max_positions": 512})}),
        "feed_forward": PartSpec("swiglu", {"hidden_size": H, "intermediate_size": inter}),
        "names": {"norm1": "input_layernorm", "mixer": "self_attn", "norm2": "post_attention_layernorm",
                  "feed_forward": "mlp"}}), name="model.layers.0")
    dev, ref = random_weights(block, dtype)
    rt = runtime(dtype)
    block.setup(rt, dev)
    n = 7
    x = torch.randn(n, H, generator=torch.Generator().manual_seed(16))
    cfg = {"head_dim": d, "rms_norm_eps": eps, "rope_theta": theta}
    once = plain.decoder_layer(x.double(), ref, 0, cfg, torch.arange(n), None)
    want = plain.decoder_layer(once, ref, 0, cfg, torch.arange(n), None)
    layout = layout_of({0: block.mixer.cache_spec(), 1: block.mixer.cache_spec()})
    norm_kernels = []
    real = ops.add_rmsnorm
    monkeypatch.setattr(ops, "add_rmsnorm", lambda *a, **k: (norm_kernels.append(1), real(*a, **k))[1])
    from qwen3_from_scratch_b200.parts.base import NEXT_NORM_WEIGHT
    # "told": the model has told the block which norm reads the stream next, so its last projection leaves the
    # stream times that weight and the next call needs no norm kernel; "not told": the next call runs its first norm
    for way in ("told", "not told", "norm kernels"):
        fused = way != "norm kernels"
        if not fused:
            monkeypatch.setattr(type(block), "fuses", lambda self, rows: False)
        manager = CacheManager(layout, 4, 64, rt.max_seqs)
        storage = CacheStorage(layout, 4, rt.max_seqs, rt.device, rt.dtype)
        manager.open("r")
        manager.reserve("r", n)
        ctx = BatchContext(manager, storage, rt).build([Entry("r", [0] * n)], vocab_size=1)
        ctx.per_step = {NEXT_NORM_WEIGHT: block.first_norm_weight} if way == "told" else {}
        stream = x.cuda().clone()
        del norm_kernels[:]
        assert block.fuses(n) == fused
        pending = block.forward(stream, None, ctx, 0, True)
        if fused:
            assert pending is None
            assert (ctx.per_step[STREAM_SUMSQ].scaled is not None) == (way == "told")
        else:
            assert pending is not None
        pending = block.forward(stream, pending, ctx, 1, True)
        assert len(norm_kernels) == {"told": 1, "not told": 2, "norm kernels": 4}[way]
        close(stream.clone() if fused else stream + pending.float(), want, dtype)
    assert int(rt.status.item()) == 0


# ---------------------------------------------------------------------- a toy mixer with state
def register_toy():
    """Registers, from the test, a mixer that keeps a decayed running sum per request in a state
    slot, and an architecture that uses it in every second layer.  Nothing in the package changes."""
    from qwen3_from_scratch_b200.config.model_config import ModelConfig
    from qwen3_from_scratch_b200.parts.base import LayerCall, Mixer, ModelSpec, PartSpec, StateSpec, WeightSpec
    from qwen3_from_scratch_b200.parts.linear import Linear
    from qwen3_from_scratch_b200.registry import register_architecture, register_part, registered_architectures

    if "ToyStateLM" in registered_architectures():
        return

    @register_part("mixer", "toy_running_sum")
    class RunningSum(Mixer):
        def __init__(self, name, hidden_size, decay):
            super().__init__(name)
            self.hidden_size, self.decay = hidden_size, decay

        def weight_specs(self):
            return [WeightSpec(f"{self.name}.proj.weight", (self.hidden_size, self.hidden_size))]

        def cache_spec(self):
            return StateSpec((self.hidden_size,), "float32")

        def setup(self, rt, weights):
            super().setup(rt, weights)
            self.proj = Linear(weights[f"{self.name}.proj.weight"], rt, tag="toy.proj")

        def forward(self, x, ctx, cache_id, write_cache):
            state = ctx.state(cache_id)  # [slots, hidden] float32
            slots = ctx.slot_ids.tolist()
            sums = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            at = 0
            for row, n in enumerate(ctx.q_lens):
                s = state[slots[row]]
                for t in range(at, at + n):
                    s = s * self.decay + x[t].float()
                    sums[t] = s
                state[slots[row]] = s
                at += n
            return self.proj(sums.to(x.dtype))

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int = 0
        width: int = 0
        depth: int = 0
        decay: float = 0.0

        @classmethod
        def from_dict(cls, data):
            return cls(data["architectures"][0], data["vocab_size"], data["width"], data["depth"], data["decay"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "width": self.width,
                    "depth": self.depth, "decay": self.decay}

    @register_architecture("ToyStateLM", ToyConfig)
    def toy_spec(cfg):
        norm = PartSpec("rms_norm", {"dim": cfg.width, "eps": 1e-5})
        ff = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": 2 * cfg.width})
        attn = PartSpec("gqa_attention", {"hidden_size": cfg.width, "num_heads": 2, "num_kv_heads": 1,
                                          "head_dim": 16, "qk_norm_eps": None, "position": None})
        toy = PartSpec("toy_running_sum", {"hidden_size": cfg.width, "decay": cfg.decay})
        layers = [(f"layers.{i}", PartSpec("pre_norm", {"norm1": norm, "norm2": norm, "feed_forward": ff,
                                                        "mixer": toy if i % 2 == 0 else attn}))
                  for i in range(cfg.depth)]
        # the run order names layer 0 twice (shared weights, a state of its own each time)
        order = [LayerCall(i, i) for i in range(cfg.depth)] + [LayerCall(0, cfg.depth)]
        return ModelSpec(embedding=("embed", PartSpec("token_embedding", {"vocab_size": cfg.vocab_size,
                                                                          "hidden_size": cfg.width})),
                         layers=layers, order=order, final_norm=("final_norm", norm),
                         head=("head", PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.width})),
                         vocab_size=cfg.vocab_size, max_positions=4096)


def toy_plain_logits(folder, ids):
    """The toy model restated with plain torch in float64 (whole sequence, no cache, no slots)."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    x = w["embed.weight"][torch.tensor(ids)]
    n = len(ids)

    def layer(x, i):
        p = f"layers.{i}"
        h = plain.rms_norm(x, w[f"{p}.norm1.weight"], 1e-5)
        if i % 2 == 0:
            s, sums = torch.zeros(cfg["width"], dtype=torch.float64), []
            for t in range(n):
                s = s * cfg["decay"] + h[t]
                sums.append(s)
            a = torch.stack(sums) @ w[f"{p}.mixer.proj.weight"].t()
        else:
            q = (h @ w[f"{p}.mixer.q_proj.weight"].t()).view(n, 2, 16)
            k = (h @ w[f"{p}.mixer.k_proj.weight"].t()).view(n, 1, 16)
            v = (h @ w[f"{p}.mixer.v_proj.weight"].t()).view(n, 1, 16)
            a = plain.causal_attention(q, k, v).reshape(n, -1) @ w[f"{p}.mixer.o_proj.weight"].t()
        x = x + a
        return x + plain.swiglu_mlp(plain.rms_norm(x, w[f"{p}.norm2.weight"], 1e-5), w, f"{p}.feed_forward")

    for i in range(cfg["depth"]):
        x = layer(x, i)
    x = layer(x, 0)
    return plain.rms_norm(x, w["final_norm.weight"], 1e-5) @ w["head.weight"].t()


def test_toy_mixer_with_state_registers_builds_and_steps(tmp_path):
    register_toy()
    from qwen3_from_scratch_b200.engine.session import Session
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    cfg = config_from_dict({"architectures": ["ToyStateLM"], "vocab_size": 97, "width": 32, "depth": 3, "decay": 0.9})
    folder = str(tmp_path / "toy")
    write_random_model(folder, cfg, seed=3)
    g = torch.Generator().manual_seed(9)
    seqs = {"x": torch.randint(0, 97, (40,), generator=g).tolist(),
            "y": torch.randint(0, 97, (23,), generator=g).tolist()}
    want = {r: toy_plain_logits(folder, ids).float() for r, ids in seqs.items()}
    session = Session(folder, dtype="float32", page_size=8, cache_tokens=256, max_seqs=4, max_step_tokens=128)
    layout = session.model.cache_layout()
    assert sorted(layout.states) == [0, 2, 3] and [g.cache_ids for g in layout.groups] == [[1]]
    # whole
    rep = Replayer(session, seqs)
    rep.step([("x", 40), ("y", 23)])
    whole = rep.result()
    # in portions, the two requests interleaved: the state has to be carried from step to step
    rep2 = Replayer(session, seqs)
    for nx, ny in [(7, 1), (1, 9), (20, 2), (12, 11)]:
        rep2.step([("x", nx), ("y", ny)])
    cut = rep2.result()
    for r in seqs:
        scale = float(want[r].abs().max())
        assert float((whole[r] - want[r]).abs().max()) <= 1e-5 * scale
        assert float((cut[r] - want[r]).abs().max()) <= 1e-5 * scale
    # a slot handed to a new request starts from zero state
    rep3 = Replayer(session, {"z": seqs["y"]})
    rep3.step([("z", 23)])
    assert float((rep3.result()["z"] - want["y"]).abs().max()) <= 1e-5 * float(want["y"].abs().max())


def register_toy_routed():
    """A second toy architecture, again defined here alone: attention with a position encoding the
    fused kernel does not know (a gain that depends on the position), and a feed-forward that routes
    every token to one of a few small experts (router logits and softmax in float32)."""
    from qwen3_from_scratch_b200.config import ModelConfig
    from qwen3_from_scratch_b200.parts.base import (FeedForward, LayerCall, ModelSpec, PartSpec, PositionEncoding,
                                                   WeightSpec)
    from qwen3_from_scratch_b200.registry import register_architecture, register_part, registered_architectures
    if "ToyRoutedLM" in registered_architectures():
        return

    @register_part("position", "toy_position_gain")
    class PositionGain(PositionEncoding):
        """y[t, h, j] = x[t, h, j] * (1 + depth * cos(position_t * rate^j))."""

        def __init__(self, name, head_dim, depth, rate):
            super().__init__(name)
            self.head_dim, self.depth, self.rate = head_dim, depth, rate

        def setup(self, rt, weights):
            super().setup(rt, weights)
            self.freq = (self.rate ** torch.arange(self.head_dim, dtype=torch.float32)).to(rt.device)

        def apply(self, x, positions):
            gain = 1 + self.depth * torch.cos(positions.float()[:, None] * self.freq[None, :])
            return (x.float() * gain[:, None, :]).to(x.dtype)

    @register_part("feed_forward", "toy_routed")
    class Routed(FeedForward):
        def __init__(self, name, hidden_size, inner, experts):
            super().__init__(name)
            self.hidden_size, self.inner, self.experts = hidden_size, inner, experts

        def weight_specs(self):
            specs = [WeightSpec(f"{self.name}.router.weight", (self.experts, self.hidden_size))]
            for e in range(self.experts):
                specs += [WeightSpec(f"{self.name}.experts.{e}.w_in.weight", (self.inner, self.hidden_size)),
                          WeightSpec(f"{self.name}.experts.{e}.w_out.weight", (self.hidden_size, self.inner))]
            return specs

        def setup(self, rt, weights):
            super().setup(rt, weights)
            self.router = weights[f"{self.name}.router.weight"]
            self.w_in = [weights[f"{self.name}.experts.{e}.w_in.weight"] for e in range(self.experts)]
            self.w_out = [weights[f"{self.name}.experts.{e}.w_out.weight"] for e in range(self.experts)]

        def forward(self, x):
            probs = torch.softmax(x.float() @ self.router.float().t(), dim=-1)
            weight, choice = probs.max(dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.experts):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(x[rows].float() @ self.w_in[e].float().t())
                    out[rows] = (h @ self.w_out[e].float().t()) * weight[rows, None]
            return out.to(x.dtype)

    @dataclass(frozen=True)
    class RoutedConfig(ModelConfig):
        vocab_size: int = 0
        width: int = 0
        depth: int = 0
        experts: int = 0

        @classmethod
        def from_dict(cls, data):
            return cls(data["architectures"][0], data["vocab_size"], data["width"], data["depth"], data["experts"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "width": self.width,
                    "depth": self.depth, "experts": self.experts}

    @register_architecture("ToyRoutedLM", RoutedConfig)
    def routed_spec(cfg):
        norm = PartSpec("rms_norm", {"dim": cfg.width, "eps": 1e-6})
        position = PartSpec("toy_position_gain", {"head_dim": 16, "depth": 0.5, "rate": 0.8})
        attn = PartSpec("gqa_attention", {"hidden_size": cfg.width, "num_heads": 4, "num_kv_heads": 2, "head_dim": 16,
                                          "qk_norm_eps": 1e-6, "position": position})
        routed = PartSpec("toy_routed", {"hidden_size": cfg.width, "inner": 24, "experts": cfg.experts})
        dense = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": 40})
        layers = [(f"layers.{i}", PartSpec("pre_norm", {"norm1": norm, "norm2": norm, "mixer": attn,
                                                        "feed_forward": routed if i % 2 == 0 else dense}))
                  for i in range(cfg.depth)]
        return ModelSpec(embedding=("embed", PartSpec("token_embedding", {"vocab_size": cfg.vocab_size,
                                                                          "hidden_size": cfg.width})),
                         layers=layers, order=[LayerCall(i, i) for i in range(cfg.depth)],
                         final_norm=("final_norm", norm),
                         head=("head", PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.width})),
                         vocab_size=cfg.vocab_size, max_positions=4096)


def routed_plain_logits(folder, ids):
    """The routed toy model in float64, whole sequence, no cache.  Returns the logits and the smallest
    margin between the two largest router probabilities (a near-tie could route differently in float32)."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    x = w["embed.weight"][torch.tensor(ids)]
    n = len(ids)
    gain = 1 + 0.5 * torch.cos(torch.arange(n, dtype=torch.float64)[:, None] * (0.8 ** torch.arange(16, dtype=torch.float64))[None, :])
    margin = 1.0
    for i in range(cfg["depth"]):
        p = f"layers.{i}"
        h = plain.rms_norm(x, w[f"{p}.norm1.weight"], 1e-6)
        q = (h @ w[f"{p}.mixer.q_proj.weight"].t()).view(n, 4, 16)
        k = (h @ w[f"{p}.mixer.k_proj.weight"].t()).view(n, 2, 16)
        v = (h @ w[f"{p}.mixer.v_proj.weight"].t()).view(n, 2, 16)
        q = plain.rms_norm(q, w[f"{p}.mixer.q_norm.weight"], 1e-6) * gain[:, None, :]
        k = plain.rms_norm(k, w[f"{p}.mixer.k_norm.weight"], 1e-6) * gain[:, None, :]
        x = x + plain.causal_attention(q, k, v).reshape(n, -1) @ w[f"{p}.mixer.o_proj.weight"].t()
        h = plain.rms_norm(x, w[f"{p}.norm2.weight"], 1e-6)
        if i % 2 == 0:
            probs = torch.softmax(h @ w[f"{p}.feed_forward.router.weight"].t(), dim=-1)
            top2 = probs.topk(2, dim=-1).values
            margin = min(margin, float((top2[:, 0] - top2[:, 1]).min()))
            weight, choice = probs.max(dim=-1)
            f = torch.zeros_like(h)
            for t in range(n):
                e = int(choice[t])
                inner = torch.relu(h[t] @ w[f"{p}.feed_forward.experts.{e}.w_in.weight"].t())
                f[t] = inner @ w[f"{p}.feed_forward.experts.{e}.w_out.weight"].t() * weight[t]
        else:
            f = plain.swiglu_mlp(h, w, f"{p}.feed_forward")
        x = x + f
    return plain.rms_norm(x, w["final_norm.weight"], 1e-6) @ w["head.weight"].t(), margin


def test_toy_routed_feed_forward_and_position_encoding(tmp_path):
    """A feed-forward with routing and a position encoding of its own, registered from this file, built
    from a configuration, loaded from a folder and stepped whole and in portions."""
    register_toy_routed()
    from qwen3_from_scratch_b200.engine.session import Session
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    cfg = config_from_dict({"architectures": ["ToyRoutedLM"], "vocab_size": 83, "width": 48, "depth": 3, "experts": 3})
    folder = str(tmp_path / "routed")
    write_random_model(folder, cfg, seed=4, dtype="float32")
    g = torch.Generator().manual_seed(10)
    seqs = {"x": torch.randint(0, 83, (37,), generator=g).tolist(), "y": torch.randint(0, 83, (18,), generator=g).tolist()}
    want = {}
    for r, ids in seqs.items():
        logits, margin = routed_plain_logits(folder, ids)
        assert margin > 1e-4  # no token sits on the fence between two experts
        want[r] = logits.float()
    session = Session(folder, dtype="float32", page_size=8, cache_tokens=256, max_seqs=4, max_step_tokens=128)
    rep = Replayer(session, seqs)
    rep.step([("x", 37), ("y", 18)])
    whole = rep.result()
    rep2 = Replayer(session, seqs)
    for nx, ny in [(5, 2), (1, 1), (19, 9), (12, 6)]:
        rep2.step([("x", nx), ("y", ny)])
    cut = rep2.result()
    for r in seqs:
        scale = float(want[r].abs().max())
        assert float((whole[r] - want[r]).abs().max()) <= 1e-5 * scale
        assert float((cut[r] - want[r]).abs().max()) <= 1e-5 * scale


# ---------------------------------------------------------------------- a toy mixer with a cache of one plane
def register_toy_latent():
    """A third toy architecture, again defined here alone.  Its mixer keeps ONE vector per token (a latent
    of a width of its own, in float32) in a paged cache with a single plane, and reads two numbers per token
    that the caller sends beside the token ids (``Entry.extra["axes"]``): it answers a token with the mean of
    the latents of all tokens so far that share the token's second number, times an output matrix."""
    from qwen3_from_scratch_b200.config import ModelConfig
    from qwen3_from_scratch_b200.parts.base import (CachePlane, LayerCall, Mixer, ModelSpec, PagedCacheSpec, PartSpec,
                                                   WeightSpec)
    from qwen3_from_scratch_b200.parts.linear import Linear
    from qwen3_from_scratch_b200.registry import register_architecture, register_part, registered_architectures
    if "ToyLatentLM" in registered_architectures():
        return

    @register_part("mixer", "toy_latent_mean")
    class LatentMean(Mixer):
        def __init__(self, name, hidden_size, latent):
            super().__init__(name)
            self.hidden_size, self.latent = hidden_size, latent

        def weight_specs(self):
            return [WeightSpec(f"{self.name}.down.weight", (self.latent, self.hidden_size)),
                    WeightSpec(f"{self.name}.up.weight", (self.hidden_size, self.latent))]

        def cache_spec(self):
            # per token: the latent and, behind it, the token's second number
            return PagedCacheSpec((CachePlane("latent", 1, self.latent + 1, "float32"),))

        def setup(self, rt, weights):
            super().setup(rt, weights)
            self.down = Linear(weights[f"{self.name}.down.weight"], rt, tag="toy.latent.down")
            self.up = Linear(weights[f"{self.name}.up.weight"], rt, tag="toy.latent.up")

        def forward(self, x, ctx, cache_id, write_cache):
            planes, table = ctx.pages(cache_id)
            pages = planes["latent"]  # [num_pages, 1, page_size, latent + 1]
            page = pages.shape[2]
            rows = table.tolist()
            second = ctx.extra["axes"][:, 1].tolist()
            lat = self.down(x).float()
            out = torch.empty_like(lat)
            at = 0
            for b, n in enumerate(ctx.q_lens):
                start = ctx.kv_lens[b] - n
                for i in range(n):
                    pos, t = start + i, at + i
                    if write_cache:
                        slot = pages[rows[b][pos // page], 0, pos % page]
                        slot[:self.latent] = lat[t]
                        slot[self.latent] = float(second[t])
                    seen = torch.stack([pages[rows[b][p // page], 0, p % page] for p in range(pos + 1)])
                    same = seen[:, self.latent] == float(second[t])
                    out[t] = seen[same, :self.latent].mean(dim=0)
                at += n
            return self.up(out.to(x.dtype))

    @dataclass(frozen=True)
    class LatentConfig(ModelConfig):
        vocab_size: int = 0
        width: int = 0
        latent: int = 0

        @classmethod
        def from_dict(cls, data):
            return cls(data["architectures"][0], data["vocab_size"], data["width"], data["latent"])

        def to_dict(self):
            return {"architectures": [self.architecture], "vocab_size": self.vocab_size, "width": self.width,
                    "latent": self.latent}

    @register_architecture("ToyLatentLM", LatentConfig)
    def latent_spec(cfg):
        norm = PartSpec("rms_norm", {"dim": cfg.width, "eps": 1e-6})
        ff = PartSpec("swiglu", {"hidden_size": cfg.width, "intermediate_size": 2 * cfg.width})
        attn = PartSpec("gqa_attention", {"hidden_size": cfg.width, "num_heads": 2, "num_kv_heads": 2,
                                          "head_dim": 16, "qk_norm_eps": None, "position": None})
        latent = PartSpec("toy_latent_mean", {"hidden_size": cfg.width, "latent": cfg.latent})
        layers = [(f"layers.{i}", PartSpec("pre_norm", {"norm1": norm, "norm2": norm, "feed_forward": ff, "mixer": m}))
                  for i, m in enumerate([latent, attn, latent])]
        return ModelSpec(embedding=("embed", PartSpec("token_embedding", {"vocab_size": cfg.vocab_size,
                                                                          "hidden_size": cfg.width})),
                         layers=layers, order=[LayerCall(i, i) for i in range(3)], final_norm=("final_norm", norm),
                         head=("head", PartSpec("lm_head", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.width})),
                         vocab_size=cfg.vocab_size, max_positions=4096)


def latent_plain_logits(folder, ids, second):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    from safetensors.torch import load_file
    w = {k: v.double() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}
    x = w["embed.weight"][torch.tensor(ids)]
    n = len(ids)
    second = torch.tensor(second)
    for i in range(3):
        p = f"layers.{i}"
        h = plain.rms_norm(x, w[f"{p}.norm1.weight"], 1e-6)
        if i != 1:
            lat = (h @ w[f"{p}.mixer.down.weight"].t()).float().double()  # the cache holds it in float32
            mean = torch.stack([lat[:t + 1][second[:t + 1] == second[t]].mean(dim=0) for t in range(n)])
            a = mean @ w[f"{p}.mixer.up.weight"].t()
        else:
            q = (h @ w[f"{p}.mixer.q_proj.weight"].t()).view(n, 2, 16)
            k = (h @ w[f"{p}.mixer.k_proj.weight"].t()).view(n, 2, 16)
            v = (h @ w[f"{p}.mixer.v_proj.weight"].t()).view(n, 2, 16)
            a = plain.causal_attention(q, k, v).reshape(n, -1) @ w[f"{p}.mixer.o_proj.weight"].t()
        x = x + a
        x = x + plain.swiglu_mlp(plain.rms_norm(x, w[f"{p}.norm2.weight"], 1e-6), w, f"{p}.feed_forward")
    return plain.rms_norm(x, w["final_norm.weight"], 1e-6) @ w["head.weight"].t()


def test_toy_mixer_with_a_one_plane_cache_and_numbers_sent_beside_the_tokens(tmp_path):
    """The cache storage gives a mixer the planes it declares (here one, wider than the model's heads, in
    float32, beside the attention layer's keys and values in a group of their own), and the step context
    carries per-token integers of the caller's to the parts; whole and in portions, two requests interleaved."""
    register_toy_latent()
    from qwen3_from_scratch_b200.engine.batch import Entry
    from qwen3_from_scratch_b200.engine.session import Session
    from qwen3_from_scratch_b200.registry import config_from_dict
    from qwen3_from_scratch_b200.weights import write_random_model
    cfg = config_from_dict({"architectures": ["ToyLatentLM"], "vocab_size": 61, "width": 32, "latent": 12})
    folder = str(tmp_path / "latent")
    write_random_model(folder, cfg, seed=6, dtype="float32")
    g = torch.Generator().manual_seed(12)
    ids = {"x": torch.randint(0, 61, (29,), generator=g).tolist(), "y": torch.randint(0, 61, (14,), generator=g).tolist()}
    axes = {r: [[t, int(v)] for t, v in enumerate(torch.randint(0, 3, (len(s),), generator=g).tolist())]
            for r, s in ids.items()}
    want = {r: latent_plain_logits(folder, ids[r], [a[1] for a in axes[r]]).float() for r in ids}
    session = Session(folder, dtype="float32", page_size=4, cache_tokens=128, max_seqs=4, max_step_tokens=64)
    layout = session.model.cache_layout()
    assert [g.cache_ids for g in layout.groups] == [[0, 2], [1]]
    assert [p.name for p in layout.groups[0].spec.planes] == ["latent"]
    assert set(session.storage.planes(0)) == {"latent"} and session.storage.planes(0)["latent"].shape[-1] == 13
    assert session.storage.planes(0)["latent"].dtype == torch.float32 and set(session.storage.planes(1)) == {"k", "v"}

    def run(cuts):
        fed = {r: 0 for r in ids}
        rows = {r: [] for r in ids}
        for cut in cuts:
            entries = []
            for r, n in cut:
                a = fed[r]
                entries.append(Entry(r, ids[r][a:a + n], list(range(n)), {"axes": axes[r][a:a + n]}))
                fed[r] += n
            logits = session.step(entries).float().cpu()
            session.check_status()
            at = 0
            for r, n in cut:
                rows[r].append(logits[at:at + n])
                at += n
        for r in ids:
            session.end(r)
        return {r: torch.cat(v) for r, v in rows.items()}

    whole = run([[("x", 29), ("y", 14)]])
    cut = run([[("x", 6), ("y", 1)], [("x", 1), ("y", 5)], [("y", 7), ("x", 13)], [("x", 9), ("y", 1)]])
    for r in ids:
        scale = float(want[r].abs().max())
        assert float((whole[r] - want[r]).abs().max()) <= 1e-5 * scale
        assert float((cut[r] - want[r]).abs().max()) <= 1e-5 * scale
    with pytest.raises(ValueError, match="per-token arrays"):
        session.step([Entry("x", ids["x"][:3], (), {"axes": axes["x"][:3]}), Entry("y", ids["y"][:3], ())])
