"""Plain, slow implementation of Qwen3 dense, the oracle of the tests.

Whole sequences, no cache, one function for each part, float32 (or float64), on the CPU or,
for models of real width, on whatever device the weights were moved to (plain torch either way).
It shares no code with the engine: it reads config.json and model.safetensors itself
(through the safetensors package) and is written from the formulas of the reference
(1483795887/qwen3_from_scratch); each function names the file and lines it follows.
Paths are relative to the reference's ``src/qwen3_from_scratch/``.

``tests/golden/`` holds logits of the reference's own model code for one tiny model;
``tests/test_plain_vs_reference.py`` checks this file against them.
"""

from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Sequence

import torch
from safetensors import safe_open


def read_model_folder(folder: str, dtype=torch.float32):
    """config.json as a dict and every tensor of model.safetensors widened to ``dtype``."""
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    weights: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for name in f.keys():
            weights[name] = f.get_tensor(name).to(dtype)
    return config, weights


def layer_windows(config: dict) -> List[Optional[int]]:
    """Per layer, the sliding window or None.  The reference ignores these keys (it has full
    attention only); their meaning here is the checkpoint format's: ``layer_types`` if given,
    else layers from ``max_window_layers`` on when ``use_sliding_window`` is set."""
    n = config["num_hidden_layers"]
    window = config.get("sliding_window")
    types = config.get("layer_types")
    if types is None:
        if config.get("use_sliding_window") and window is not None:
            first = config.get("max_window_layers", n)
            types = ["sliding_attention" if i >= first else "full_attention" for i in range(n)]
        else:
            types = ["full_attention"] * n
    return [window if t == "sliding_attention" else None for t in types]


# ---------------------------------------------------------------------- parts
def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """x[t] = E[ids[t]], no scaling (models/qwen3.py:17-19,45)."""
    return table[ids.long()]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w over the last dimension
    (models/norm.py:18-22 with F.rms_norm; csrc/rms_norm/rms_norm.cpp:13-31)."""
    mean_sq = x.pow(2).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(mean_sq + eps) * weight


def rope_cos_sin(positions: torch.Tensor, head_dim: int, theta: float, dtype=torch.float32):
    """cos/sin of position * theta^(-2j/D), j < D/2 (models/rotary.py:36-45).  The inverse
    frequencies and the angle are formed in float32 as there, then widened if asked."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=positions.device) / head_dim))
    freqs = torch.einsum("i,j->ij", positions.to(torch.float32), inv_freq)
    return freqs.cos().to(dtype), freqs.sin().to(dtype)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half: y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin on the two halves of the head
    (models/rotary.py:13-22).  x: [T, heads, D]; cos, sin: [T, D/2]."""
    x1, x2 = torch.chunk(x, 2, dim=-1)
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat((x1 * c - x2 * s, x2 * c + x1 * s), dim=-1)


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: Optional[int] = None) -> torch.Tensor:
    """Whole-sequence grouped-query attention.  q: [T, Hq, D]; k, v: [T, Hkv, D].
    q head h reads kv head h // (Hq / Hkv); scores (q.k) * D^-0.5; key n visible to query m
    when n <= m (models/attn.py:388-400 for the scale, :452-456 for the mask, :421 for the
    head mapping) and, with a window, n > m - window."""
    T, hq, d = q.shape
    hkv = k.shape[1]
    g = hq // hkv
    scale = d ** -0.5
    m_idx = torch.arange(T, device=q.device)[:, None]
    n_idx = torch.arange(T, device=q.device)[None, :]
    hidden = n_idx > m_idx
    if window is not None:
        hidden = hidden | (n_idx <= m_idx - window)
    out = torch.empty_like(q)
    for h in range(hq):
        scores = (q[:, h] @ k[:, h // g].t()) * scale
        scores = scores.masked_fill(hidden, float("-inf"))
        out[:, h] = torch.softmax(scores, dim=-1) @ v[:, h // g]
    return out


def self_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str, config: dict,
                   positions: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """q/k/v projections, per-head RMSNorm of q and k, rotation, attention, output projection
    (models/self_attn.py:41-58 and :310-342: norm before rotation, v untouched, no biases)."""
    T = x.shape[0]
    d = config["head_dim"]
    eps = config["rms_norm_eps"]
    q = (x @ w[f"{prefix}.q_proj.weight"].t()).view(T, -1, d)
    k = (x @ w[f"{prefix}.k_proj.weight"].t()).view(T, -1, d)
    v = (x @ w[f"{prefix}.v_proj.weight"].t()).view(T, -1, d)
    q = rms_norm(q, w[f"{prefix}.q_norm.weight"], eps)
    k = rms_norm(k, w[f"{prefix}.k_norm.weight"], eps)
    cos, sin = rope_cos_sin(positions, d, float(config["rope_theta"]), dtype=x.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    o = causal_attention(q, k, v, window)
    return o.reshape(T, -1) @ w[f"{prefix}.o_proj.weight"].t()


def swiglu_mlp(x: torch.Tensor, w: Dict[str, torch.Tensor], prefix: str) -> torch.Tensor:
    """down(up(x) * silu(gate(x))) (models/feedback.py:28-34)."""
    up = x @ w[f"{prefix}.up_proj.weight"].t()
    gate = x @ w[f"{prefix}.gate_proj.weight"].t()
    return (up * (gate * torch.sigmoid(gate))) @ w[f"{prefix}.down_proj.weight"].t()


def decoder_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], i: int, config: dict,
                  positions: torch.Tensor, window: Optional[int]) -> torch.Tensor:
    """h = x + attn(norm(x)); y = h + mlp(norm(h)) (models/transformer_block.py:38-46)."""
    p = f"model.layers.{i}"
    eps = config["rms_norm_eps"]
    h = x + self_attention(rms_norm(x, w[f"{p}.input_layernorm.weight"], eps), w, f"{p}.self_attn", config,
                           positions, window)
    return h + swiglu_mlp(rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], eps), w, f"{p}.mlp")


def lm_head(h: torch.Tensor, w: Dict[str, torch.Tensor], config: dict) -> torch.Tensor:
    """logits = h W^T with the embedding table when tied (models/qwen3.py:63-74,83-84)."""
    table = w["model.embed_tokens.weight"] if config.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return h @ table.t()


def forward_logits(config: dict, w: Dict[str, torch.Tensor], ids: Sequence[int]) -> torch.Tensor:
    """Logits at every position of one whole sequence, [T, vocab] (models/qwen3.py:44-50,80-84)."""
    device = w["model.embed_tokens.weight"].device
    ids = torch.as_tensor(list(ids), dtype=torch.long, device=device)
    positions = torch.arange(ids.numel(), device=device)
    x = embedding(ids, w["model.embed_tokens.weight"])
    for i, window in enumerate(layer_windows(config)):
        x = decoder_layer(x, w, i, config, positions, window)
    x = rms_norm(x, w["model.norm.weight"], config["rms_norm_eps"])
    return lm_head(x, w, config)


# ---------------------------------------------------------------------- sampling
_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = (z + 0x9E3779B97F4A7C15) & _M64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def sample_uniforms(seed: int, request_key: int, position: int, n: int) -> torch.Tensor:
    """The engine's documented generator, restated: u_i in (0, 1) for i < n, float32."""
    row_key = _mix64((_mix64(seed & _M64) + _mix64(request_key & _M64) * 3 + (position & _M64)) & _M64)
    vals = [((_mix64((row_key + i) & _M64) >> 41) + 0.5) * 2.0 ** -23 for i in range(n)]
    return torch.tensor(vals, dtype=torch.float32)


def greedy_token(logits: torch.Tensor) -> int:
    """argmax (inference/sampler.py:17-21); the lowest id among equals."""
    return int(torch.argmax(logits.float()))


def sample_token(logits: torch.Tensor, temperature: float, top_k: int, seed: int, request_key: int,
                 position: int) -> int:
    """A draw from softmax(logits / T) (inference/sampler.py:24-33), among the top_k largest when
    top_k > 0 (:36-56), in the Gumbel-max form with the generator above: the same distribution
    as softmax + multinomial, and the same token as the engine for the same key."""
    logits = logits.float()
    if temperature <= 0:
        return greedy_token(logits)
    u = sample_uniforms(seed, request_key, position, logits.numel())
    gumbel = -torch.log(-torch.log(u))
    scores = logits / torch.tensor(temperature, dtype=torch.float32) + gumbel
    if 0 < top_k < logits.numel():
        kth = torch.topk(logits, top_k).values[-1]
        scores = scores.masked_fill(logits < kth, float("-inf"))
    return int(torch.argmax(scores))
