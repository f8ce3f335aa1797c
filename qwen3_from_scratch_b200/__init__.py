"""A single-GPU inference engine for the Qwen3 dense architecture on NVIDIA B200 (sm_100a).

From a model folder (config.json + safetensors) to generated tokens: typed configuration and
architecture registry, weights by tensor name, layers assembled from parameterised parts, a
paged cache manager, one step function over mixed batches, a continuous-batching scheduler,
sampling, and hand-written CUDA kernels.  See ``engine.Engine`` for the Python entry point
and ``cli`` for the command line.
"""

__version__ = "0.1.0"
