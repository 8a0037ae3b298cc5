"""Arrangements of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.specs import BlockSpec
from .base import Block, ParamSpec, build_feed_forward, build_mixer, build_norm, register_block


class AssembledBlock(Block):
    """A block put together from child parts.  ``children()`` says which: a dict from slot name to
    part, in a fixed order; parameters, loading and the capture flag walk it, so an arrangement with
    more parts (a norm after a branch, a third branch) overrides ``children`` and ``forward`` and
    nothing else.  A parameter's key is "<slot>/<the child's own key>".  This base builds the usual
    four from the spec: ``norm``, ``mixer``, ``ffn`` and, if the spec has one, ``norm2``."""

    def __init__(self, spec: BlockSpec):
        self.spec = spec
        self.norm = build_norm(spec.norm)
        self.norm2 = build_norm(spec.norm2) if spec.norm2 is not None else None
        self.mixer = build_mixer(spec.mixer)
        self.ffn = build_feed_forward(spec.ffn)

    def children(self) -> Dict[str, object]:
        c = {"norm": self.norm}
        if self.norm2 is not None:
            c["norm2"] = self.norm2
        c["mixer"] = self.mixer
        c["ffn"] = self.ffn
        return c

    def parameters(self) -> Dict[str, ParamSpec]:
        return {f"{slot}/{k}": v for slot, part in self.children().items() for k, v in part.parameters().items()}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        for slot, part in self.children().items():
            pre = slot + "/"
            part.load({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})

    def cache_request(self):
        return self.mixer.cache_request()

    def products(self):
        return [(f"{slot}.{name}", w, b, act) for slot, part in self.children().items()
                for name, w, b, act in part.products()]

    @property
    def capturable(self):
        return all(part.capturable for part in self.children().values())

    @property
    def launches_only(self):
        return all(part.launches_only for part in self.children().values())


class ParallelBlock(AssembledBlock):
    """x ← (x + ffn(n)) + mixer(n), n = norm(x): one norm feeds both branches
    (model.go:2738-2740) and both are added to the residual, the feed-forward
    first (model.go:2812-2815)."""

    def _decode_step_as_one_kernel(self, x, ctx, cache) -> bool:
        """With one token a sequence a layer is a stream of weights and cached keys and values; where
        every part offers its fused form and the kernel takes the sizes, the whole block runs as one
        persistent kernel that keeps that stream going from the norm to the residual sum."""
        if not (ctx.is_decode and ctx.act_dtype == torch.bfloat16 and self.norm.fusable is not None
                and self.mixer.decode_fusable is not None and self.ffn.fusable is not None):
            return False
        m = self.mixer.decode_fusable(ctx, cache)
        if m is None:
            return False
        w_up, b_up, act, w_down, b_down = self.ffn.fusable()
        half = 0 if m["cos"] is None else m["cos"].shape[1]
        if not ops.decode_layer_takes(x, m["w_qkv"], w_up, m["w_out"], w_down, m["k"].dtype, m["head_dim"],
                                      m["num_heads"] // m["num_kv_heads"], half, m["interleaved"], m["head_norm"],
                                      longest=ctx.max_len):
            return False
        g, b, eps, rms = self.norm.fusable()
        ops.decode_layer(x, g, b, eps, rms, m["w_qkv"], m["b_qkv"], w_up, b_up, act, m["w_out"], m["b_out"],
                         w_down, b_down, m["k"], m["v"], ctx.seq_ctx, m["pages"], m["num_heads"], m["num_kv_heads"],
                         m["head_dim"], m["q_scale"], m["cos"], m["sin"], m["window"], m["writes"])
        return True

    def forward(self, x, ctx, cache):
        if self._decode_step_as_one_kernel(x, ctx, cache):
            return x
        xn = self.norm.forward(x, ctx.act_dtype)
        side = getattr(ctx, "side_stream", None)
        if self.ffn.until_last is not None and self.mixer.until_last is not None:
            # The branches' last products end on the same rows and columns: they run as one product
            # over the joined K where the kernels can (one kernel, one pass over the residual stream),
            # else one after the other.  What comes before them runs on two streams in decode steps:
            # with few tokens every kernel is a stream of weights, and the feed-forward's first product
            # keeps memory busy while the mixer's small kernels start and finish.
            if side is None and self.ffn.first_product is not None and self.mixer.first_product is not None:
                # many tokens: the branches' first products read the same rows and run as one grid
                wm, bm, am = self.mixer.first_product()
                wf, bf, af = self.ffn.first_product()
                ym, yf = ops.linear_fork(xn, wm, bm, am, wf, bf, af, ctx.act_dtype)
                h, w2, b2 = self.ffn.until_last(xn, ctx, first=yf)
                o, wo, bo = self.mixer.until_last(xn, ctx, cache, first=ym)
            elif side is None:
                h, w2, b2 = self.ffn.until_last(xn, ctx)
                o, wo, bo = self.mixer.until_last(xn, ctx, cache)
            else:
                main = torch.cuda.current_stream()
                fork, join = torch.cuda.Event(), torch.cuda.Event()
                fork.record(main)
                side.wait_event(fork)
                with torch.cuda.stream(side):
                    h, w2, b2 = self.ffn.until_last(xn, ctx)
                    join.record(side)
                o, wo, bo = self.mixer.until_last(xn, ctx, cache)
                main.wait_event(join)
            ops.linear_pair(h, w2, b2, o, wo, bo, add0=x, out=x)
            return x
        if side is None or not self.mixer.deferred_add:
            # each branch adds itself onto the residual stream in its last product's epilogue,
            # the feed-forward first: (x + mlp) + attn, the reference's order
            self.ffn.forward(xn, ctx, (x,), x)
            self.mixer.forward(xn, ctx, cache, (x,), x)
            return x
        # Both branches read the same normalised input, so the feed-forward runs on a second
        # stream beside the mixer and leaves its result in a buffer of its own; the mixer's last
        # product adds both the residual and that buffer.  With few tokens every kernel is a
        # stream of weights: the second stream keeps memory busy while the mixer's small kernels
        # start and finish, and nothing of the feed-forward is left on the path from one layer's
        # norm to the next.  The sum is the same three terms in 32-bit, added as (attn + x) + mlp.
        main = torch.cuda.current_stream()
        y = ops.empty(x.shape, torch.float32, x.device)
        fork, join = torch.cuda.Event(), torch.cuda.Event()
        fork.record(main)
        side.wait_event(fork)
        with torch.cuda.stream(side):
            self.ffn.forward(xn, ctx, (), y)
            join.record(side)
        def mlp():                   # resolved by the mixer just before its last product
            main.wait_event(join)
            return y

        self.mixer.forward(xn, ctx, cache, (x, mlp), x)
        return x


class SequentialBlock(AssembledBlock):
    """x ← x + mixer(norm(x)); x ← x + ffn(norm2(x)) (model.go:2806-2811)."""

    def __init__(self, spec: BlockSpec):
        if spec.norm2 is None:
            raise ValueError("a sequential block needs norm2")
        super().__init__(spec)

    def forward(self, x, ctx, cache):
        self.mixer.forward(self.norm.forward(x, ctx.act_dtype), ctx, cache, (x,), x)
        self.ffn.forward(self.norm2.forward(x, ctx.act_dtype), ctx, (x,), x)
        return x


register_block("parallel", ParallelBlock)
register_block("sequential", SequentialBlock)
