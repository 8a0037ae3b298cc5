"""Feed-forward parts."""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from .. import ops
from ..config.specs import FeedForwardSpec
from .base import FeedForward, ParamSpec, register_feed_forward


class DenseFeedForward(FeedForward):
    """down(act(up(x))) with biases: the plain, ungated MLP (model.go:2758-2772,
    forward_batch.go:537-581).  The activation runs in the first product's
    epilogue, the additions to the residual in the second's."""
    capturable = True
    launches_only = True

    def __init__(self, spec: FeedForwardSpec):
        if spec.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {spec.activation!r} unknown")
        self.spec = spec
        self.w_up = self.b_up = self.w_down = self.b_down = None

    def parameters(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p = {"up.weight": ParamSpec((s.intermediate, s.hidden)),
             "down.weight": ParamSpec((s.hidden, s.intermediate))}
        if s.bias:
            p["up.bias"] = ParamSpec((s.intermediate,), "vector", "bias")
            p["down.bias"] = ParamSpec((s.hidden,), "vector", "bias")
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.w_up, self.w_down = t["up.weight"], t["down.weight"]
        self.b_up, self.b_down = t.get("up.bias"), t.get("down.bias")

    def first_product(self):
        return self.w_up, self.b_up, self.spec.activation

    def fusable(self):
        return self.w_up, self.b_up, self.spec.activation, self.w_down, self.b_down

    def products(self):
        return [("up", self.w_up, self.b_up, self.spec.activation), ("down", self.w_down, self.b_down, None)]

    def until_last(self, xn, ctx, first=None):
        h = first if first is not None else ops.linear(xn, self.w_up, self.b_up, act=self.spec.activation,
                                                       out_dtype=ctx.act_dtype)
        return h, self.w_down, self.b_down

    def forward(self, xn, ctx, add: Sequence[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        if len(add) > 2:
            raise ValueError("at most two tensors can be added in the projection's epilogue")
        h = ops.linear(xn, self.w_up, self.b_up, act=self.spec.activation, out_dtype=ctx.act_dtype)
        a0 = add[0] if len(add) > 0 else None
        a1 = add[1] if len(add) > 1 else None
        return ops.linear(h, self.w_down, self.b_down, add0=a0, add1=a1, out=out)


register_feed_forward("dense", DenseFeedForward)
