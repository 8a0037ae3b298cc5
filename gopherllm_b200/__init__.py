"""gopherllm_b200: a small, whole model library for one B200.

From a model folder (config.json + model.safetensors) to generated tokens:
typed configuration and architecture registry, weights by name, layers built
from parts, a paged cache with slots, one batched step function, a generation
loop with sampling, and trace replay, on hand-written sm_100a kernels in
bfloat16 and in true 32-bit.
"""
from .api import LoadInfo, Model, load, load_random, write_random_model
from .engine.generate import (GenerationCanceled, GenerationOptions, GenerationResult,
                              GenerationStats)
from .sampling.sampler import PRESETS, SamplerConfig

__version__ = "0.1.0"
__all__ = ["load", "load_random", "write_random_model", "Model", "LoadInfo", "GenerationOptions",
           "GenerationResult", "GenerationStats", "GenerationCanceled", "SamplerConfig", "PRESETS"]
