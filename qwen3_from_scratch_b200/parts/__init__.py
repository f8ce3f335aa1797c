"""Parts a model is put together from.  ``parts.base`` holds the interfaces; the built-in
parts live in the sibling modules and are registered when the registry is first used."""

from .base import (Block, CachePlane, FeedForward, KVCacheSpec, LayerCall, Mixer, ModelSpec, Norm,  # noqa: F401
                   PagedCacheSpec, Part, PartSpec, PositionEncoding, Runtime, StateSpec, StepContext, WeightSpec)
