"""Interfaces of the parts a layer is put together from, and their registries.

A part is built from its spec alone (sizes and constants as parameters), says
which tensors it owns (``parameters``), takes them (``load``) and computes
(``forward``).  It never learns which model it sits in.  New kinds are added
with ``register_norm`` / ``register_position`` / ``register_mixer`` /
``register_feed_forward`` / ``register_block`` and are then chosen by the
``kind`` (or ``arrangement``) field of a spec, layer by layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch


@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part owns.

    kind: "matrix" (kept in the stored 16/32-bit type), "vector" (held in
    float32: the reference reads every 1-D tensor as float32, model.go:2519-2528)
    or "table_int" (held as int32).
    init: how the random-weights mode fills it: "normal" N(0, initializer_range),
    "bias"/"beta" N(0, 0.02), "gamma" 1 + N(0, 0.02), "zeros".
    optional: a missing tensor is replaced by zeros (model.go:2229-2231).
    """
    shape: Tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"
    optional: bool = False


@dataclass(frozen=True)
class KVRequest:
    """A mixer's need for cached keys and values: per position ``num_kv_heads``
    rows of ``head_dim``; ``window`` 0 keeps every position, w > 0 the last w."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateRequest:
    """A mixer's need for per-sequence state of fixed size (float32), zeroed
    when a sequence starts (the reference zeroes such state at request start
    because it is read before it is written, runtime.go:1526-1539)."""
    shape: Tuple[int, ...]


class Part:
    """Common protocol of every part.

    capturable: True if ``forward`` only launches work on the current stream (no copy to
    the host, no host-side decision on device data), so a step can be recorded into a
    CUDA graph.  The default is False: a part must opt in.

    launches_only: True if everything ``forward`` does on the device is a launch through
    ``gopherllm_b200.ops`` (no torch operation, no copy, no second stream) with memory from
    ``ops.empty``, and what it does on the host does not depend on which of several equal parts
    it is.  A model repeats the recorded launches of such a block for the next equal block
    instead of walking through its parts again.  The default is False: a part must opt in.
    """
    capturable = False
    launches_only = False

    def parameters(self) -> Dict[str, ParamSpec]:
        return {}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Take ownership of the tensors named in ``parameters`` (already on the
        device and in the types ParamSpec.kind promises)."""
        for k, v in tensors.items():
            setattr(self, "p_" + k.replace(".", "_"), v)

    def products(self) -> List[Tuple[str, torch.Tensor, Optional[torch.Tensor], Optional[str]]]:
        """The matrix products this part makes for every token, as (name, weight [out, in], bias,
        activation), in the order it makes them; for measurement (flop counts, isolated kernel
        timing) by code that does not know the part's kind.  Parts may leave it empty."""
        return []


class Norm(Part):
    """forward(x float32 [R, D], out_dtype, rows=None) -> [R', D] of out_dtype.
    Optional: ``fusable()`` -> (weight, bias or None, eps, rms) for a block that runs its decode step
    as one kernel; a norm without it is simply run through ``forward``."""
    fusable = None

    def forward(self, x: torch.Tensor, out_dtype: torch.dtype, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        raise NotImplementedError


class PositionEncoding(Part):
    """Per-step tables for a mixer.  ``tables(ctx)`` may cache in ctx.scratch."""

    def tables(self, ctx):
        raise NotImplementedError


class Mixer(Part):
    """Token mixer.

    cache_request(): KVRequest, StateRequest or None.
    forward(xn, ctx, cache, add, out): out = mix(xn) + sum(add), float32 [T, hidden].
      xn   [T, hidden] in ctx.act_dtype, the normalised input
      cache: the view the cache built for this run's entry (None if no request)
      add  : float32 tensors of out's shape to add (the residual stream and/or
             another branch); out may alias one of them
    """

    def cache_request(self):
        return None

    # Optional: ``until_last(xn, ctx, cache)`` -> (activations, weight, bias), everything but the last
    # product, for a block that runs the last products of its branches as one (ops.linear_pair).
    until_last = None
    # Optional, with until_last: ``first_product()`` -> (weight, bias, activation) of the product that
    # until_last starts with on xn; until_last then takes ``first=`` that product's result instead of
    # computing it, so that a block can run the first products of its branches as one (ops.linear_fork).
    first_product = None

    # Optional: ``decode_fusable(ctx, cache)`` -> a dict describing a one-token-a-sequence step of softmax
    # attention over the paged cache (w_qkv, b_qkv, w_out, b_out, num_heads, num_kv_heads, head_dim, q_scale,
    # window, cos, sin, interleaved, head_norm, k, v, pages, writes), or None when this step is not of
    # that kind; a block whose parts all offer the fused form may run its decode step as one kernel.
    decode_fusable = None

    # A mixer that sets this accepts callables among ``add``: it calls them just before its last
    # product and adds what they return.  A block uses that to let another branch run beside the
    # mixer on a second stream and join only where its result is needed.
    deferred_add = False

    def forward(self, xn, ctx, cache, add: Sequence[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    """forward(xn, ctx, add, out): out = ffn(xn) + sum(add), float32 [T, hidden].
    Optional: until_last(xn, ctx) -> (activations, weight, bias), everything but the last product;
    with it, first_product() -> (weight, bias, activation) and until_last(..., first=result), as for a mixer."""

    until_last = None
    first_product = None
    # Optional: ``fusable()`` -> (w_up, b_up, activation, w_down, b_down) of a plain two-product feed-forward.
    fusable = None

    def forward(self, xn, ctx, add: Sequence[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block(Part):
    """One layer: owns a norm (or two), a mixer and a feed-forward and runs them
    in its arrangement.  forward(x, ctx, cache) updates the float32 residual
    stream x [T, hidden] in place."""

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


_NORMS: Dict[str, Callable] = {}
_POSITIONS: Dict[str, Callable] = {}
_MIXERS: Dict[str, Callable] = {}
_FEED_FORWARDS: Dict[str, Callable] = {}
_BLOCKS: Dict[str, Callable] = {}


def _register(table: Dict[str, Callable], what: str):
    def reg(kind: str, factory: Callable, replace: bool = False) -> None:
        if kind in table and not replace:
            raise ValueError(f"{what} kind {kind!r} is already registered")
        table[kind] = factory
    return reg


def _build(table: Dict[str, Callable], what: str):
    def make(spec, *args, **kw):
        kind = getattr(spec, "kind", None) or getattr(spec, "arrangement", None)
        if kind not in table:
            raise ValueError(f"unknown {what} kind {kind!r} (known: {', '.join(sorted(table))})")
        return table[kind](spec, *args, **kw)
    return make


register_norm = _register(_NORMS, "norm")
register_position = _register(_POSITIONS, "position encoding")
register_mixer = _register(_MIXERS, "mixer")
register_feed_forward = _register(_FEED_FORWARDS, "feed-forward")
register_block = _register(_BLOCKS, "block")
build_norm = _build(_NORMS, "norm")
build_position = _build(_POSITIONS, "position encoding")
build_mixer = _build(_MIXERS, "mixer")
build_feed_forward = _build(_FEED_FORWARDS, "feed-forward")
build_block = _build(_BLOCKS, "block")
