"""Softmax attention over the paged key/value cache."""
from __future__ import annotations

from typing import Dict, Sequence

import torch

from .. import ops
from ..config.specs import MixerSpec
from .base import KVRequest, Mixer, ParamSpec, build_norm, build_position, register_mixer


class Attention(Mixer):
    """q, k, v projections (one fused product, rows ordered Q, K, V as the
    reference's fused matrix is, model.go:2222-2227), optional per-head norm of
    q and k, position encoding, query scale, cache write, attention over the
    cache, output projection.  Grouped-query attention when num_kv_heads <
    num_heads (query head h reads group h / (nH/nKV), model.go:2828)."""

    deferred_add = True
    capturable = True
    launches_only = True

    def __init__(self, spec: MixerSpec):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if spec.head_dim > 256:
            raise ValueError(f"head size {spec.head_dim} exceeds what the attention kernels take (256)")
        self.spec = spec
        self.position = build_position(spec.position)
        self.q_norm = build_norm(spec.qk_norm) if spec.qk_norm else None
        self.k_norm = build_norm(spec.qk_norm) if spec.qk_norm else None
        self.w_qkv = self.b_qkv = self.w_out = self.b_out = None

    # -- parameters -----------------------------------------------------
    def parameters(self) -> Dict[str, ParamSpec]:
        s = self.spec
        q, kv = s.num_heads * s.head_dim, s.num_kv_heads * s.head_dim
        p = {"q.weight": ParamSpec((q, s.hidden)), "k.weight": ParamSpec((kv, s.hidden)),
             "v.weight": ParamSpec((kv, s.hidden)), "out.weight": ParamSpec((s.hidden, q))}
        if s.bias:
            p.update({"q.bias": ParamSpec((q,), "vector", "bias"),
                      "k.bias": ParamSpec((kv,), "vector", "bias"),
                      "v.bias": ParamSpec((kv,), "vector", "bias"),
                      "out.bias": ParamSpec((s.hidden,), "vector", "bias")})
        if self.q_norm is not None:
            for name, n in (("q_norm", self.q_norm), ("k_norm", self.k_norm)):
                for k, v in n.parameters().items():
                    p[f"{name}.{k}"] = v
        return p

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        ws = [t["q.weight"], t["k.weight"], t["v.weight"]]
        if len({w.dtype for w in ws}) > 1:           # mixed storage: widen to the widest
            ws = [w.float() for w in ws]
        self.w_qkv = torch.cat(ws, dim=0).contiguous()
        self.w_out = t["out.weight"]
        if self.spec.bias:
            self.b_qkv = torch.cat([t["q.bias"], t["k.bias"], t["v.bias"]]).contiguous()
            self.b_out = t["out.bias"]
        if self.q_norm is not None:
            self.q_norm.load({k[len("q_norm."):]: v for k, v in t.items() if k.startswith("q_norm.")})
            self.k_norm.load({k[len("k_norm."):]: v for k, v in t.items() if k.startswith("k_norm.")})

    def cache_request(self):
        s = self.spec
        return KVRequest(s.num_kv_heads, s.head_dim, s.window)

    # -- compute ----------------------------------------------------------
    def forward(self, xn, ctx, cache, add: Sequence[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
        if len(add) > 2:
            raise ValueError("at most two tensors can be added in the projection's epilogue")
        o, w, b = self.until_last(xn, ctx, cache)
        add = [a() if callable(a) else a for a in add]
        a0 = add[0] if len(add) > 0 else None
        a1 = add[1] if len(add) > 1 else None
        return ops.linear(o, w, b, add0=a0, add1=a1, out=out)

    def first_product(self):
        return self.w_qkv, self.b_qkv, None

    def products(self):
        return [("qkv", self.w_qkv, self.b_qkv, None), ("out", self.w_out, self.b_out, None)]

    def decode_fusable(self, ctx, cache):
        if not ctx.is_decode or cache is None:
            return None
        s = self.spec
        tables = self.position.tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        return dict(w_qkv=self.w_qkv, b_qkv=self.b_qkv, w_out=self.w_out, b_out=self.b_out,
                    num_heads=s.num_heads, num_kv_heads=s.num_kv_heads, head_dim=s.head_dim, q_scale=s.q_scale,
                    window=s.window, cos=cos, sin=sin, interleaved=s.position.interleaved,
                    head_norm=self.q_norm is not None, k=cache.k, v=cache.v, pages=ctx.pages[cache.group],
                    writes=cache.writes)

    def until_last(self, xn, ctx, cache, first=None):
        """Everything but the output projection: the attention output [T, heads * head size] with the
        projection's weight and bias.  ``first``: the joined q, k, v projection if the caller made it."""
        s = self.spec
        T = xn.shape[0]
        qkv = first if first is not None else ops.linear(xn, self.w_qkv, self.b_qkv, out_dtype=ctx.act_dtype)
        tables = self.position.tables(ctx)
        cos, sin = tables if tables is not None else (None, None)
        pages = ctx.pages[cache.group]
        group = s.num_heads // s.num_kv_heads
        if (ctx.is_decode and group <= ops.DECODE_MAX_GROUP
                and ops.decode_takes_qkv(qkv.dtype, cache.k.dtype, s.head_dim, 0 if cos is None else cos.shape[1],
                                         s.position.interleaved, self.q_norm is not None)):
            # one token a sequence: attention reads the projection's output itself (rotation, query scale
            # and the cache write happen inside it), one kernel less between two products
            o = ops.empty((T, s.num_heads * s.head_dim), ctx.act_dtype, xn.device)
            splits = ops.decode_splits(ctx.n_seqs, s.num_kv_heads, ctx.max_len, xn.device, s.head_dim, group)
            ops.attention_decode(None, o, cache.k, cache.v, ctx.seq_ctx, pages, s.num_heads, s.num_kv_heads,
                                 s.head_dim, splits, s.window, qkv=qkv, cos=cos, sin=sin, q_scale=s.q_scale,
                                 write_kv=cache.writes)
            return o, self.w_out, self.b_out
        q = ops.empty((T, s.num_heads * s.head_dim), ctx.act_dtype, xn.device)
        qn = kn = None
        eps, rms = 0.0, False
        if self.q_norm is not None:
            qn, kn = (self.q_norm.weight, self.q_norm.bias), (self.k_norm.weight, self.k_norm.bias)
            eps, rms = s.qk_norm.eps, self.q_norm.rms
        ops.qkv_to_cache(qkv, q, cache.k, cache.v, ctx.tok_seq, ctx.tok_pos, pages,
                         s.num_heads, s.num_kv_heads, s.head_dim, s.q_scale, cos, sin,
                         interleaved=s.position.interleaved, q_norm=qn, k_norm=kn,
                         norm_eps=eps, norm_rms=rms, write_kv=cache.writes)
        o = ops.empty(q.shape, q.dtype, q.device)
        ops.attention(q, o, cache.k, cache.v, ctx, pages, s.num_heads, s.num_kv_heads,
                      s.head_dim, window=s.window)
        return o, self.w_out, self.b_out



register_mixer("attention", Attention)
