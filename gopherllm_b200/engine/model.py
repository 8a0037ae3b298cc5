"""A decoder model as data plus parts: embedding, the scheduled runs of its
blocks, the final norm and the output head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.specs import ModelSpec
from ..parts.base import ParamSpec, build_block, build_norm


class DecoderModel:
    """Built from a ModelSpec alone.  One block per entry of ``spec.layers``;
    ``spec.schedule`` says which block runs when and on which cache entry, so a
    block may run twice or read an entry another run wrote."""

    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.blocks = [build_block(b) for b in spec.layers]
        self.final_norm = build_norm(spec.final_norm)
        self.embedding: Optional[torch.Tensor] = None
        self.positions: Optional[torch.Tensor] = None          # learned absolute positions, if the spec has them
        self.head_weight: Optional[torch.Tensor] = None
        self.head_bias: Optional[torch.Tensor] = None

    # -- parameters -------------------------------------------------------
    def parameters(self) -> Dict[str, ParamSpec]:
        s = self.spec
        p: Dict[str, ParamSpec] = {"embedding": ParamSpec((s.vocab, s.hidden))}
        for i, b in enumerate(self.blocks):
            for k, v in b.parameters().items():
                p[f"layers/{i}/{k}"] = v
        if s.position_table:
            p["positions"] = ParamSpec((s.position_table, s.hidden))
        for k, v in self.final_norm.parameters().items():
            p[f"final_norm/{k}"] = v
        if not s.tie_embeddings:
            p["head/weight"] = ParamSpec((s.vocab, s.hidden))
        if s.head_bias:
            # with tied embeddings a file may lack the bias: zeros then
            p["head/bias"] = ParamSpec((s.vocab,), "vector", "bias", optional=s.tie_embeddings)
        return p

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.embedding = tensors["embedding"]
        self.positions = tensors["positions"] if self.spec.position_table else None
        for i, b in enumerate(self.blocks):
            pre = f"layers/{i}/"
            b.load({k[len(pre):]: v for k, v in tensors.items() if k.startswith(pre)})
        self.final_norm.load({k[len("final_norm/"):]: v for k, v in tensors.items()
                              if k.startswith("final_norm/")})
        self.head_weight = self.embedding if self.spec.tie_embeddings else tensors["head/weight"]
        self.head_bias = tensors.get("head/bias")

    @property
    def capturable(self) -> bool:
        """True if a step of this model can be recorded into a CUDA graph."""
        return self.final_norm.capturable and all(b.capturable for b in self.blocks)

    def weight_bytes(self) -> int:
        seen, n = set(), 0
        for t in self._all_tensors():
            if t is not None and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        return n

    def _all_tensors(self):
        yield self.embedding
        yield self.positions
        yield self.head_weight
        yield self.head_bias
        stack = list(self.blocks) + [self.final_norm]
        while stack:
            part = stack.pop()
            for v in vars(part).values():
                if isinstance(v, torch.Tensor):
                    yield v
                elif hasattr(v, "parameters") and hasattr(v, "load"):
                    stack.append(v)

    # -- cache --------------------------------------------------------------
    def cache_requests(self) -> List:
        """What each cache entry must hold: the request of the block whose run writes it."""
        reqs: List = [None] * self.spec.num_cache_entries
        for e in self.spec.schedule:
            if e.cache is not None and e.writes:
                reqs[e.cache] = self.blocks[e.layer].cache_request()
        for e in self.spec.schedule:
            if e.cache is not None and not e.writes:
                want, have = self.blocks[e.layer].cache_request(), reqs[e.cache]
                if want != have:
                    raise ValueError(f"layer {e.layer} reads cache entry {e.cache} but needs {want}, "
                                     f"the entry holds {have}")
        return reqs

    # -- compute ------------------------------------------------------------
    def forward(self, ctx, cache) -> torch.Tensor:
        """Run the step described by ctx; float32 logits [len(ctx.want_rows), vocab]."""
        x = self.begin(ctx)
        self.run(x, ctx, cache, 0, len(self.spec.schedule))
        return self.finish(x, ctx)

    # The same step in three pieces, for a caller that captures it as more than one CUDA graph.
    def begin(self, ctx) -> torch.Tensor:
        """The residual stream of the step's tokens, float32 [tokens, hidden]."""
        x = ops.embed(self.embedding, ctx.tokens, self.spec.embedding_scale)
        if self.positions is not None:
            ops.add_rows(self.positions, ctx.tok_pos, x)
        return x

    def run(self, x, ctx, cache, start: int, stop: int) -> None:
        """Runs start..stop-1 of the schedule, updating x in place."""
        for e in self.spec.schedule[start:stop]:
            view = cache.view(e.cache, e.writes) if e.cache is not None else None
            self.blocks[e.layer].forward(x, ctx, view)

    def finish(self, x, ctx) -> torch.Tensor:
        s = self.spec
        if ctx.n_want == 0:
            return torch.empty((0, s.vocab), dtype=torch.float32, device=x.device)
        xn = self.final_norm.forward(x, ctx.act_dtype, rows=ctx.want_rows)
        logits = ops.linear(xn, self.head_weight, self.head_bias, out_dtype=torch.float32)
        if s.logit_scale != 1.0 or s.logit_softcap > 0.0:
            ops.scale_softcap(logits, s.logit_scale, s.logit_softcap)
        return logits
