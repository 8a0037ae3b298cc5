"""Architecture-neutral descriptions of a decoder model.

A model is data: a list of block specifications (one per distinct layer), each
naming its norm, mixer, feed-forward and position encoding with all sizes and
constants, plus a schedule that says in which order layers run and which cache
entry each run uses.  Parts are built from these records and never see which
architecture produced them.

The reference keeps the same facts as predicates on one flat ``Config``
(model.go:204-319: usesLayerNorm, forcesParallelResidual,
sharesParallelBranchNorm, usesPlainMLP, layerUsesRoPE); here they are fields.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """A normalisation over the last axis.

    kind: registered norm name ("layernorm": mean/variance with bias,
    bert.go:748-776; "rmsnorm": root-mean-square, model.go:2949-2981).
    """
    kind: str
    dim: int
    eps: float
    bias: bool = True


@dataclass(frozen=True)
class PositionSpec:
    """Position encoding applied to queries and keys inside a mixer.

    kind "rope": rotary embedding over the first ``rotary_dim`` dims of each
    head; ``interleaved`` False pairs dim i with i+rotary_dim/2 (the NeoX
    split-half layout, model.go:3072-3080), True pairs 2i with 2i+1
    (model.go:3064-3071).  kind "none": nothing.
    """
    kind: str = "none"
    rotary_dim: int = 0
    theta: float = 10000.0
    interleaved: bool = False
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form options for other encodings

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class MixerSpec:
    """Token mixer of a block.  kind "attention" is softmax attention over a
    key/value cache with ``num_kv_heads`` groups; ``window`` 0 means all keys,
    w > 0 means the last w keys (the query's own position included)."""
    kind: str
    hidden: int
    num_heads: int = 0
    num_kv_heads: int = 0
    head_dim: int = 0
    window: int = 0
    q_scale: float = 1.0          # multiplies q after position encoding
    bias: bool = True
    qk_norm: Optional[NormSpec] = None
    position: PositionSpec = PositionSpec()
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form options for other mixers

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class FeedForwardSpec:
    """Feed-forward of a block.  kind "dense": act(x·W1ᵀ+b1)·W2ᵀ+b2."""
    kind: str
    hidden: int
    intermediate: int = 0
    activation: str = "gelu_new"
    bias: bool = True
    extra: Tuple[Tuple[str, object], ...] = ()

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class BlockSpec:
    """One layer.  arrangement "parallel": one norm feeds mixer and
    feed-forward, both are added to the residual (model.go:2732-2746,
    2812-2815).  arrangement "sequential": norm → mixer → add → norm2 →
    feed-forward → add."""
    arrangement: str
    norm: NormSpec
    mixer: MixerSpec
    ffn: FeedForwardSpec
    norm2: Optional[NormSpec] = None
    extra: Tuple[Tuple[str, object], ...] = ()   # free-form options for other arrangements (further norms, branches)

    def option(self, key, default=None):
        return dict(self.extra).get(key, default)


@dataclass(frozen=True)
class ScheduleEntry:
    """One run of a layer.  ``layer`` indexes ModelSpec.layers; ``cache`` is
    the cache entry this run reads (None: the mixer keeps nothing);
    ``writes`` False lets a run read an entry another run filled."""
    layer: int
    cache: Optional[int]
    writes: bool = True


@dataclass(frozen=True)
class ModelSpec:
    hidden: int
    vocab: int
    max_positions: int
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    tie_embeddings: bool = False
    head_bias: bool = True
    embedding_scale: float = 1.0
    stop_tokens: Tuple[int, ...] = ()
    # learned absolute positions: a table of this many rows added to the embeddings before the first
    # layer (model.go:2648-2651); 0: none
    position_table: int = 0
    # logits * logit_scale, then softcap * tanh(logits / softcap) when softcap > 0 (model.go:2555-2564)
    logit_scale: float = 1.0
    logit_softcap: float = 0.0

    def __post_init__(self):
        if self.position_table and self.position_table < self.max_positions:
            raise ValueError(f"a position table of {self.position_table} rows does not cover "
                             f"{self.max_positions} positions")
        if self.logit_softcap < 0 or not self.logit_scale > 0:
            raise ValueError("logit_softcap must be >= 0 and logit_scale > 0")
        for e in self.schedule:
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule names layer {e.layer}, model has {len(self.layers)}")
        writers = {}
        for e in self.schedule:
            if e.cache is None:
                continue
            if e.writes:
                if e.cache in writers:
                    raise ValueError(f"cache entry {e.cache} is written by two runs")
                writers[e.cache] = e.layer
        for e in self.schedule:
            if e.cache is not None and not e.writes and e.cache not in writers:
                raise ValueError(f"cache entry {e.cache} is read but never written")

    @property
    def num_cache_entries(self) -> int:
        ids = [e.cache for e in self.schedule if e.cache is not None]
        return (max(ids) + 1) if ids else 0


def default_schedule(num_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Layer i runs once, in order, on cache entry i."""
    return tuple(ScheduleEntry(layer=i, cache=i) for i in range(num_layers))
