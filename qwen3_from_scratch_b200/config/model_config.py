"""Typed model configuration, read from the architecture's own ``config.json`` keys.

The reference reads a fixed set of required keys with ``data[...]`` and a few
optional ones with ``data.get`` (factory/config.py:107-130).  This module keeps
the same required set and the same key names, adds the keys a Qwen3 folder
carries that the reference silently ignores (``attention_bias``,
``sliding_window`` and friends, ``rope_scaling``) and *rejects* values the
engine does not implement instead of ignoring them.

Nothing here knows a model size: every number comes from the file.
"""

from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Mapping, Optional, Tuple

FULL_ATTENTION = "full_attention"
SLIDING_ATTENTION = "sliding_attention"


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type, or names an option that is not built."""


def _require(data: Mapping[str, Any], key: str, kind):
    if key not in data:
        raise ConfigError(f"config.json: required key '{key}' is missing")
    value = data[key]
    if kind is int:
        if isinstance(value, bool) or not isinstance(value, int):
            raise ConfigError(f"config.json: '{key}' must be an integer, got {value!r}")
    elif kind is float:
        if isinstance(value, bool) or not isinstance(value, (int, float)):
            raise ConfigError(f"config.json: '{key}' must be a number, got {value!r}")
        value = float(value)
    elif kind is str:
        if not isinstance(value, str):
            raise ConfigError(f"config.json: '{key}' must be a string, got {value!r}")
    return value


def _positive(key: str, value) -> None:
    if value <= 0:
        raise ConfigError(f"config.json: '{key}' must be positive, got {value!r}")


@dataclass(frozen=True)
class ModelConfig:
    """Base of every architecture's configuration.

    ``architecture`` is the name the registry resolves (``architectures[0]`` in
    config.json).  Subclasses add the architecture's own keys.
    """

    architecture: str

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "ModelConfig":  # pragma: no cover - abstract
        raise NotImplementedError

    def to_dict(self) -> dict:
        """The config.json content that ``from_dict`` reads back to an equal object."""
        raise NotImplementedError

    def save(self, folder: str) -> str:
        path = os.path.join(folder, "config.json")
        with open(path, "w") as f:
            json.dump(self.to_dict(), f, indent=2)
            f.write("\n")
        return path


@dataclass(frozen=True)
class Qwen3Config(ModelConfig):
    """Qwen3 dense decoder (reference: models/qwen3.py:9-84, factory/config.py:19-61).

    Key names are those of the checkpoint's config.json.  ``layer_types`` is the
    per-layer mixer choice: every layer is ``full_attention`` unless the file
    turns the sliding window on.
    """

    vocab_size: int = 0
    hidden_size: int = 0
    num_hidden_layers: int = 0
    num_attention_heads: int = 0
    num_key_value_heads: int = 0
    head_dim: int = 0
    intermediate_size: int = 0
    hidden_act: str = "silu"
    rms_norm_eps: float = 0.0
    rope_theta: float = 0.0
    max_position_embeddings: int = 0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    sliding_window: Optional[int] = None
    layer_types: Tuple[str, ...] = field(default_factory=tuple)
    eos_token_id: Optional[int] = None
    bos_token_id: Optional[int] = None
    torch_dtype: str = "bfloat16"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "Qwen3Config":
        archs = data.get("architectures")
        if not isinstance(archs, (list, tuple)) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: 'architectures' must be a non-empty list of names")
        # Required exactly as in the reference's load_from_file (factory/config.py:107-130);
        # head_dim alone may be absent, then it is hidden_size / heads.
        vocab_size = _require(data, "vocab_size", int)
        hidden_size = _require(data, "hidden_size", int)
        hidden_act = _require(data, "hidden_act", str)
        num_hidden_layers = _require(data, "num_hidden_layers", int)
        max_position_embeddings = _require(data, "max_position_embeddings", int)
        num_key_value_heads = _require(data, "num_key_value_heads", int)
        num_attention_heads = _require(data, "num_attention_heads", int)
        intermediate_size = _require(data, "intermediate_size", int)
        rms_norm_eps = _require(data, "rms_norm_eps", float)
        rope_theta = _require(data, "rope_theta", float)
        for key, value in (
            ("vocab_size", vocab_size), ("hidden_size", hidden_size),
            ("num_hidden_layers", num_hidden_layers),
            ("max_position_embeddings", max_position_embeddings),
            ("num_key_value_heads", num_key_value_heads),
            ("num_attention_heads", num_attention_heads),
            ("intermediate_size", intermediate_size),
            ("rms_norm_eps", rms_norm_eps), ("rope_theta", rope_theta),
        ):
            _positive(key, value)
        if "head_dim" in data and data["head_dim"] is not None:
            head_dim = _require(data, "head_dim", int)
            _positive("head_dim", head_dim)
        else:
            if hidden_size % num_attention_heads:
                raise ConfigError(
                    "config.json: 'head_dim' is absent and hidden_size "
                    f"{hidden_size} is not a multiple of num_attention_heads {num_attention_heads}")
            head_dim = hidden_size // num_attention_heads
        if num_attention_heads % num_key_value_heads:
            raise ConfigError(
                f"config.json: num_attention_heads {num_attention_heads} is not a multiple of "
                f"num_key_value_heads {num_key_value_heads}")
        if head_dim % 2:
            raise ConfigError(f"config.json: 'head_dim' {head_dim} must be even for rotary pairs")
        if hidden_act != "silu":
            raise ConfigError(
                f"config.json: hidden_act '{hidden_act}' is not built (only 'silu', "
                "as in the reference's activation_map)")
        if data.get("attention_bias", False):
            raise ConfigError("config.json: attention_bias=true is not built (Qwen3 dense has none)")
        scaling = data.get("rope_scaling")
        if scaling not in (None, {}):
            raise ConfigError(f"config.json: rope_scaling {scaling!r} is not built (plain rotary only)")

        # ---- per-layer mixer choice
        window = data.get("sliding_window")
        if window is not None:
            if isinstance(window, bool) or not isinstance(window, int) or window <= 0:
                raise ConfigError(f"config.json: 'sliding_window' must be a positive integer or null, got {window!r}")
        layer_types = data.get("layer_types")
        if layer_types is not None:
            if not isinstance(layer_types, (list, tuple)) or len(layer_types) != num_hidden_layers:
                raise ConfigError(
                    f"config.json: 'layer_types' must list {num_hidden_layers} layers, got {layer_types!r}")
            for t in layer_types:
                if t not in (FULL_ATTENTION, SLIDING_ATTENTION):
                    raise ConfigError(f"config.json: layer type {t!r} is not built")
            layer_types = tuple(layer_types)
        elif data.get("use_sliding_window", False) and window is not None:
            # The first max_window_layers layers keep full attention, the rest use the window.
            first_windowed = data.get("max_window_layers", num_hidden_layers)
            if isinstance(first_windowed, bool) or not isinstance(first_windowed, int) or first_windowed < 0:
                raise ConfigError(f"config.json: 'max_window_layers' must be a non-negative integer, got {first_windowed!r}")
            layer_types = tuple(
                SLIDING_ATTENTION if i >= first_windowed else FULL_ATTENTION
                for i in range(num_hidden_layers))
        else:
            layer_types = (FULL_ATTENTION,) * num_hidden_layers
        if SLIDING_ATTENTION in layer_types and window is None:
            raise ConfigError("config.json: a layer is 'sliding_attention' but 'sliding_window' is null")
        if SLIDING_ATTENTION not in layer_types:
            window = None

        eos = data.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else None
        return cls(
            architecture=archs[0],
            vocab_size=vocab_size, hidden_size=hidden_size,
            num_hidden_layers=num_hidden_layers,
            num_attention_heads=num_attention_heads,
            num_key_value_heads=num_key_value_heads,
            head_dim=head_dim, intermediate_size=intermediate_size,
            hidden_act=hidden_act, rms_norm_eps=rms_norm_eps, rope_theta=rope_theta,
            max_position_embeddings=max_position_embeddings,
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            attention_bias=False, sliding_window=window, layer_types=layer_types,
            eos_token_id=eos, bos_token_id=data.get("bos_token_id"),
            torch_dtype=str(data.get("torch_dtype", data.get("dtype", "bfloat16"))),
        )

    # ------------------------------------------------------------------ writing
    def to_dict(self) -> dict:
        d = asdict(self)
        arch = d.pop("architecture")
        d["architectures"] = [arch]
        d["model_type"] = "qwen3"
        d["layer_types"] = list(self.layer_types)
        d["use_sliding_window"] = self.sliding_window is not None
        d["rope_scaling"] = None
        return d


def read_config_json(folder_or_file: str) -> dict:
    """The raw config.json of a model folder."""
    path = folder_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.isfile(path):
        raise ConfigError(f"no config.json at {path}")
    with open(path) as f:
        try:
            data = json.load(f)
        except json.JSONDecodeError as e:
            raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(data, dict):
        raise ConfigError(f"{path}: top level must be an object")
    return data
