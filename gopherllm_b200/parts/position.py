"""Position encodings a mixer can be given."""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..config.specs import PositionSpec
from .base import PositionEncoding, register_position


def rope_inverse_frequencies(rotary_dim: int, theta: float) -> np.ndarray:
    """inv[i] = 1 / float32(theta ** float32(2i / rotary_dim)); the exponent is a
    32-bit quotient, the power is taken in 64-bit and rounded to 32-bit
    (buildRopeInvFreq, model.go:1742-1750)."""
    half = rotary_dim // 2
    i = (np.arange(half, dtype=np.float32) * np.float32(2.0))
    e = i / np.float32(rotary_dim)
    base = np.power(np.float64(theta), e.astype(np.float64)).astype(np.float32)
    return (np.float32(1.0) / base).astype(np.float32)


class Rope(PositionEncoding):
    """Rotary embedding over the first ``rotary_dim`` dims of a head.  The
    angle float32(pos) * inv[i] is a 32-bit product; sine and cosine are taken
    in 64-bit (prepareRopeScratch, model.go:3041-3046).  The tables depend on
    the step's positions only, so every layer of a step shares them."""
    capturable = True
    launches_only = True

    def __init__(self, spec: PositionSpec):
        if spec.rotary_dim % 2:
            raise ValueError(f"rotary dimension {spec.rotary_dim} must be even")
        self.spec = spec
        self._inv = None

    def tables(self, ctx):
        key = ("rope", self.spec.rotary_dim, float(self.spec.theta))
        hit = ctx.scratch.get(key)
        if hit is None:
            if self._inv is None or self._inv.device != ctx.device:
                self._inv = torch.from_numpy(
                    rope_inverse_frequencies(self.spec.rotary_dim, self.spec.theta)).to(ctx.device)
            hit = ops.rope_table(ctx.tok_pos, self._inv)
            ctx.scratch[key] = hit
        return hit


class NoPosition(PositionEncoding):
    capturable = True
    launches_only = True
    def __init__(self, spec: PositionSpec):
        self.spec = spec

    def tables(self, ctx):
        return None


register_position("rope", Rope)
register_position("none", NoPosition)
