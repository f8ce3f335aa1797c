"""Parts a model is put together from.  ``parts.base`` holds the interfaces; the built-in
parts live in the sibling modules and are registered when the registry is first used."""

from .base import (Block, FeedForward, KVCacheSpec, LayerCall, Mixer, ModelSpec, Norm, Part, PartSpec,  # noqa: F401
                   PositionEncoding, Runtime, StateSpec, StepContext, WeightSpec)
