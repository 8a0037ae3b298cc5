"""Sampler options and the per-batch sampler state on the device.

Options, defaults and rules are the reference's SamplerConfig (sampling.go:48-61:
temperature 0.7, top_p 0.9, top_k 40, min_p 0, repeat_penalty 1.1; disabled
values top_k <= 0, top_p >= 1, min_p <= 0, repeat_penalty == 1; temperature 0 is
greedy) and GenerationOptions.Validate (runtime.go:166-192).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional, Sequence

import torch

from .. import ops

WINDOW = ops.SAMPLE_WINDOW
_ZERO_SEED = 0xDEADBEEFCAFE1337      # xorshift has an all-zero fixed point (sampling.go:30-35)
_MASK64 = (1 << 64) - 1


@dataclass
class SamplerConfig:
    temperature: float = 0.7
    top_p: float = 0.9
    top_k: int = 40
    min_p: float = 0.0
    repeat_penalty: float = 1.1

    @classmethod
    def greedy(cls) -> "SamplerConfig":
        """The reference's "deterministic" preset (cmd/gopherllm/config.go:330)."""
        return cls(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, repeat_penalty=1.0)

    @property
    def is_greedy(self) -> bool:
        return self.temperature < 1e-6 or self.top_k == 1

    def validate(self) -> None:
        def finite(v):
            return isinstance(v, (int, float)) and math.isfinite(v)
        if not finite(self.temperature) or self.temperature < 0:
            raise ValueError("temperature must be a finite number >= 0")
        if not finite(self.top_p) or self.top_p <= 0 or self.top_p > 1:
            raise ValueError("top_p must be in the range (0, 1]")
        if not isinstance(self.top_k, int) or self.top_k < 0:
            raise ValueError("top_k must be greater than or equal to 0")
        if not finite(self.min_p) or self.min_p < 0 or self.min_p > 1:
            raise ValueError("min_p must be in the range [0, 1]")
        if not finite(self.repeat_penalty) or self.repeat_penalty <= 0:
            raise ValueError("repeat_penalty must be a finite number > 0")


PRESETS = {
    # cmd/gopherllm/config.go:317-336
    "balanced": SamplerConfig(),
    "precise": SamplerConfig(0.2, 0.9, 30, 0.0, 1.05),
    "creative": SamplerConfig(0.95, 0.95, 80, 0.05, 1.05),
    "deterministic": SamplerConfig.greedy(),
}


def request_seed(seed: int, index: int) -> int:
    """Generator state of request ``index`` of a call seeded with ``seed``: each
    request has a generator of its own, so its draws do not depend on what else
    is in the batch.  A state of zero is remapped (sampling.go:30-35)."""
    s = (int(seed) + int(index)) & _MASK64
    return s if s != 0 else _ZERO_SEED


def recent_window(tokens: Sequence[int]) -> List[int]:
    """The trailing window the repeat penalty starts from: the prompt's last 64
    tokens (recentTokenWindowInto, runtime.go:1225)."""
    return list(tokens[-WINDOW:])


class DeviceSampler:
    """Sampler state of a batch of requests on the device: one generator state
    and one window of recent tokens per request."""

    def __init__(self, config: SamplerConfig, seeds: Sequence[int], prompts: Sequence[Sequence[int]],
                 vocab: int, device):
        config.validate()
        ops.check_sampler(config.temperature, config.top_k, config.top_p, config.min_p, vocab)
        self.config, self.vocab, self.device = config, vocab, device
        n = len(seeds)
        self.n = n
        recent = torch.zeros((n, WINDOW), dtype=torch.int32)
        recent_n = torch.zeros(n, dtype=torch.int32)
        for i, p in enumerate(prompts):
            w = recent_window(p)
            recent[i, :len(w)] = torch.tensor(w, dtype=torch.int32)
            recent_n[i] = len(w)
        signed = [s - (1 << 64) if s >= (1 << 63) else s for s in seeds]
        self.rng = torch.tensor(signed, dtype=torch.int64).to(device)
        self.recent = recent.to(device)
        self.recent_n = recent_n.to(device)
        self.out = torch.zeros(n, dtype=torch.int32, device=device)
        self.work = torch.empty((n, vocab), dtype=torch.float32, device=device)
        self.sort_key = self.sort_idx = None
        if ops.needs_sort_scratch(config.temperature, config.top_k, config.top_p, config.min_p, vocab):
            vpad = ops.sort_scratch_size(vocab)
            self.sort_key = torch.empty((n, vpad), dtype=torch.float32, device=device)
            self.sort_idx = torch.empty((n, vpad), dtype=torch.int32, device=device)

    def sample(self, logits: torch.Tensor, state_row: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Tokens [B] int32 (a view of an internal buffer) for logits [B, V]."""
        c = self.config
        B = logits.shape[0]
        ops.sample(logits, self.work, self.recent, self.recent_n, self.rng, self.out,
                   c.temperature, c.top_k, c.top_p, c.min_p, c.repeat_penalty, state_row=state_row,
                   sort_key=self.sort_key, sort_idx=self.sort_idx)
        return self.out[:B]
