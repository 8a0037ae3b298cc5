"""A decoder model as data plus parts: embedding, the scheduled runs of its
blocks, the final norm and the output head."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.specs import ModelSpec
from ..parts.base import ParamSpec, build_block, build_norm


def _tensor_addresses(part, prefix: str) -> Dict[str, int]:
    """name -> address (0 for None) of the tensors an object holds as attributes, in lists, tuples and
    dicts, and inside the parts it holds; names are attribute paths, so equal for equal parts."""
    out: Dict[str, int] = {}

    def walk(v, name, depth):
        if isinstance(v, torch.Tensor):
            out[name] = v.data_ptr()
        elif isinstance(v, (list, tuple)):
            for i, u in enumerate(v):
                walk(u, f"{name}[{i}]", depth)
        elif isinstance(v, dict):
            for k, u in v.items():
                walk(u, f"{name}[{k!r}]", depth)
        elif hasattr(v, "parameters") and hasattr(v, "load") and depth < 8:
            for k, u in sorted(vars(v).items()):
                walk(u, f"{name}.{k}", depth + 1)

    for k, v in sorted(vars(part).items()):
        walk(v, prefix + k, 0)
    return out


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
        self._held: Dict[int, Dict[str, int]] = {}             # layer -> addresses of its tensors (see run)

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
        self._held = {}

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
        """Runs start..stop-1 of the schedule, updating x in place.

        The layers of a model are mostly the same block with other tensors, and what the host does
        for one run of a block (the parts' choices, checks, argument records) costs more time than
        the kernels of a short prompt take.  So the launches of a block's run are recorded, compared
        with the launches of the next run of an equal block (they must be the same but for the two
        blocks' own tensors and temporaries), and from the third such run on repeated with that
        run's tensors in place of the recorded ones.  Runs that fork onto a second stream are left
        alone: their events are no launches."""
        repeat = ops.REPEAT_LAYERS and getattr(ctx, "side_stream", None) is None and stop - start > 2
        kinds: List[list] = []            # [block, writes, view type, tape, pointers, state, tries]
        for e in self.spec.schedule[start:stop]:
            view = cache.view(e.cache, e.writes) if e.cache is not None else None
            block = self.blocks[e.layer]
            if not repeat or not getattr(block, "launches_only", False):
                block.forward(x, ctx, view)
                continue
            ptrs = self._pointers(e.layer, view)
            kind = next((k for k in kinds if type(k[0]) is type(block) and k[0].spec == block.spec
                         and k[1] == e.writes and k[2] is type(view)), None)
            if kind is not None and kind[5] == "repeat":
                kind[3].repeat(ptrs)
                continue
            if kind is not None and kind[5] == "own":
                block.forward(x, ctx, view)
                continue
            tape = ops.LaunchTape().start()
            try:
                block.forward(x, ctx, view)
            finally:
                tape.stop()
            if kind is None:
                kinds.append([block, e.writes, type(view), tape, ptrs, "recorded", 0])
            elif kind[3].same_as(tape, kind[4], ptrs):
                kind[3].bind(kind[4])
                kind[5] = "repeat"
            else:
                # (the first run of a step may do what later ones find done: tables of the step's
                # positions, say; so the later run becomes the one to compare with, a few times)
                kind[3], kind[4], kind[6] = tape, ptrs, kind[6] + 1
                if kind[6] >= 3:
                    kind[5] = "own"

    def _pointers(self, layer: int, view) -> Dict[str, int]:
        """name -> address of every tensor block ``layer`` holds, and of the cache entry it runs on."""
        held = self._held.get(layer)
        if held is None:
            held = self._held[layer] = _tensor_addresses(self.blocks[layer], "")
        if view is None:
            return held
        ptrs = dict(held)
        ptrs.update(_tensor_addresses(view, "cache/"))
        return ptrs

    def finish(self, x, ctx) -> torch.Tensor:
        s = self.spec
        if ctx.n_want == 0:
            return torch.empty((0, s.vocab), dtype=torch.float32, device=x.device)
        xn = self.final_norm.forward(x, ctx.act_dtype, rows=ctx.want_rows)
        logits = ops.linear(xn, self.head_weight, self.head_bias, out_dtype=torch.float32)
        if s.logit_scale != 1.0 or s.logit_softcap > 0.0:
            ops.scale_softcap(logits, s.logit_scale, s.logit_softcap)
        return logits
