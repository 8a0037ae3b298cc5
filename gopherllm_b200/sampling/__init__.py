from .sampler import PRESETS, DeviceSampler, SamplerConfig, recent_window, request_seed
