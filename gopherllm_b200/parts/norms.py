"""Normalisation parts: LayerNorm and RMSNorm over the last axis."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from ..config.specs import NormSpec
from .base import Norm, ParamSpec, register_norm


class LayerNorm(Norm):
    """y = (x - mean) * rsqrt(var + eps) * weight + bias, biased variance, in
    32-bit with the reciprocal square root in 64-bit (bert.go:748-776)."""
    capturable = True
    launches_only = True
    rms = False

    def __init__(self, spec: NormSpec):
        self.spec = spec
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def parameters(self) -> Dict[str, ParamSpec]:
        p = {"weight": ParamSpec((self.spec.dim,), "vector", "gamma")}
        if self.spec.bias:
            p["bias"] = ParamSpec((self.spec.dim,), "vector", "beta")
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"]
        self.bias = tensors.get("bias")

    def fusable(self):
        return self.weight, self.bias, self.spec.eps, self.rms

    def forward(self, x, out_dtype, rows=None):
        return ops.norm(x, self.weight, self.bias, self.spec.eps, out_dtype, rms=self.rms, rows=rows)


class RMSNorm(LayerNorm):
    """y = x * rsqrt(mean(x²) + eps) * weight (model.go:2949-2981)."""
    rms = True


register_norm("layernorm", LayerNorm)
register_norm("rmsnorm", RMSNorm)
