"""The model as the engine runs it: parts built from a ModelSpec, and the step function.

``Model.step(ctx)`` runs exactly the tokens of the batch, reading and writing the caches
the context hands out, and returns float32 logits at the rows the batch asks for
(the reference's worker instead samples a token for every sequence, including those
still in their prompt: inference/model_worker.py:212-227).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..cache.manager import CacheLayout, layout_of
from ..config.model_config import ModelConfig
from ..kernels import ops
from ..parts.base import NEXT_NORM_WEIGHT, STREAM_SUMSQ, ModelSpec, Runtime, StepContext
from ..registry import build_model_spec, create_part, load_config
from ..weights.loader import load_weights
from ..weights.random_init import random_weights_on_device

DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine computes in bfloat16 or float32, not {dtype}")
        return dtype
    try:
        return DTYPES[str(dtype).lower()]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, got '{dtype}'") from None


class Model:
    def __init__(self, spec: ModelSpec):
        """Builds the parts (no device work yet): ``weight_specs`` and ``cache_layout`` are available."""
        self.spec = spec
        emb_name, emb = spec.embedding
        self.embedding = create_part("embedding", emb, name=emb_name)
        self.layers = [create_part("block", block, name=name) for name, block in spec.layers]
        norm_name, norm = spec.final_norm
        self.final_norm = create_part("norm", norm, name=norm_name)
        head_name, head = spec.head
        self.head = create_part("head", head, name=head_name)
        for i, call in enumerate(spec.order):
            if not 0 <= call.layer < len(self.layers):
                raise ValueError(f"run order entry {i} names layer {call.layer}, the model has {len(self.layers)}")
        self.rt: Optional[Runtime] = None

    @property
    def graph_capturable(self) -> bool:
        return all(p.graph_capturable for p in [self.embedding, self.final_norm, self.head] + self.layers)

    def weight_specs(self):
        specs = list(self.embedding.weight_specs())
        for layer in self.layers:
            specs += layer.weight_specs()
        specs += self.final_norm.weight_specs()
        specs += self.head.weight_specs()
        return specs

    def cache_layout(self) -> CacheLayout:
        """What every cache id of the run order has to hold, as its writer's mixer asks."""
        needs: Dict[int, object] = {}
        for call in self.spec.order:
            if call.cache is None:
                continue
            need = self.layers[call.layer].mixer.cache_spec()
            if call.cache in needs:
                if needs[call.cache] != need:
                    raise ValueError(f"cache {call.cache} is used by layers with different needs")
                if call.write_cache:
                    raise ValueError(f"cache {call.cache} has two writers in the run order")
            elif not call.write_cache:
                raise ValueError(f"cache {call.cache} is read before any layer wrote it")
            needs[call.cache] = need
        return layout_of(needs)

    def setup(self, rt: Runtime, weights: Dict[str, torch.Tensor]) -> None:
        self.rt = rt
        self.embedding.setup(rt, weights)
        for layer in self.layers:
            layer.setup(rt, weights)
        self.final_norm.setup(rt, weights)
        self.head.setup(rt, weights)

    @torch.inference_mode()
    def step(self, ctx: StepContext) -> torch.Tensor:
        """One batch through every layer of the run order; float32 logits [len(logit_rows), vocab]."""
        ctx.per_step = {}  # what parts share within a step is computed anew (and so is recorded by a graph capture)
        stream = self.embedding.forward(ctx.token_ids)
        pending = None
        order = self.spec.order
        for i, call in enumerate(order):
            layer = self.layers[call.layer]
            # the weight of the norm that reads the stream after this layer, for layers that prepare the stream for it
            nxt = self.layers[order[i + 1].layer] if i + 1 < len(order) else None
            ctx.per_step[NEXT_NORM_WEIGHT] = getattr(nxt, "first_norm_weight", None)
            pending = layer.forward(stream, pending, ctx, call.cache, call.write_cache)
            if not layer.keeps_stream_stats:
                ctx.per_step.pop(STREAM_SUMSQ, None)  # whatever it did to the stream, the sums describe it no longer
        if ctx.logit_rows.numel() == 0:
            return torch.empty(0, self.spec.vocab_size, dtype=torch.float32, device=stream.device)
        wanted = self.final_norm.norm_rows(stream, pending, ctx.logit_rows)
        return self.head.forward(wanted)


def load_model(folder: str, dtype, device, max_tokens: int, max_seqs: int, random_weights: Optional[int] = None):
    """config.json -> configuration -> specification -> parts -> weights on the device.
    Returns (model, configuration, runtime).  ``random_weights``: a seed; the folder then needs only its
    config.json and the weights are drawn on the device instead of read."""
    if not torch.cuda.is_available():
        raise RuntimeError("this engine runs on a CUDA GPU (sm_100a); no GPU is visible")
    ops.library()  # build or load the kernels first: without them nothing below can run
    config: ModelConfig = load_config(folder)
    model = Model(build_model_spec(config))
    compute = resolve_dtype(dtype)
    device = torch.device(device)
    rt = Runtime(device=device, dtype=compute, max_tokens=int(max_tokens), max_seqs=int(max_seqs))
    if random_weights is not None:
        weights = random_weights_on_device(model.weight_specs(), int(random_weights), device, compute)
    else:
        weights = load_weights(folder, model.weight_specs(), device=device, compute_dtype=compute,
                               ignorable=model.spec.ignorable_weights)
    model.setup(rt, weights)
    return model, config, rt
