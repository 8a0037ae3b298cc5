"""A plain, slow implementation of the Phi architecture on the CPU.

Whole sequences, no cache, no batching, one function per part, written from the
formulas of SimonWaldherr/GopherLLM (file:line at each function).  It imports
nothing from gopherllm_b200.  The reference is Go and no Go toolchain exists on
the machines this was written on, so this file rests on the reference's
formulas, not on a run of its code.

Arithmetic is float64 unless the reference rounds to 32-bit at a place where
that matters (rotary frequencies and angles); pass dtype=torch.float32 to get
32-bit arithmetic throughout.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch


# --------------------------------------------------------------------------
# model folder -> (config dict, {name: float64 tensor})
# --------------------------------------------------------------------------
def read_folder(folder, dtype=torch.float64):
    """config.json and every tensor of model.safetensors, widened to ``dtype``.
    Own small reader of the container: 8-byte length, JSON table, raw data."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    path = os.path.join(folder, "model.safetensors")
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        table = json.loads(f.read(n))
        data = f.read()
    kinds = {"F32": torch.float32, "BF16": torch.bfloat16, "F16": torch.float16, "F64": torch.float64}
    out = {}
    for name, info in table.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        t = torch.frombuffer(bytearray(data[b:e]), dtype=kinds[info["dtype"]]).reshape(info["shape"])
        out[name] = t.to(dtype)
    return cfg, out


def sizes(cfg):
    nh = cfg["num_attention_heads"]
    nkv = cfg.get("num_key_value_heads") or nh
    hd = cfg.get("head_dim") or cfg["hidden_size"] // nh
    rot = int(cfg.get("partial_rotary_factor", 0.5) * hd)
    return nh, nkv, hd, rot


# --------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------
def embedding(tokens, table):
    """x = E[token, :], no scale (model.go:2642-2651; EmbeddingScale is 1 for phi2, model.go:358-368)."""
    return table[torch.as_tensor(tokens, dtype=torch.long)]


def layer_norm(x, weight, bias, eps):
    """mean, biased variance, (x-mean) * 1/sqrt(var+eps) * w + b over the last axis
    (layerNormInto, bert.go:748-776)."""
    mean = x.sum(-1, keepdim=True) / x.shape[-1]
    d = x - mean
    var = (d * d).sum(-1, keepdim=True) / x.shape[-1]
    scale = 1.0 / torch.sqrt(var + eps)
    return d * scale * weight + (bias if bias is not None else 0.0)


def rope_inv_freq(rotary_dim, theta):
    """inv[i] = 1/float32(theta ** float32(2i/R)) (buildRopeInvFreq, model.go:1742-1750)."""
    inv = []
    for pair in range(rotary_dim // 2):
        e = np.float32(pair * 2) / np.float32(rotary_dim)
        base = np.float32(math.pow(float(theta), float(e)))
        inv.append(np.float32(1.0) / base)
    return np.array(inv, dtype=np.float32)


def rope_tables(positions, rotary_dim, theta):
    """sin/cos of float64(float32(pos) * inv[i]) rounded to float32
    (prepareRopeScratch, model.go:3041-3046)."""
    inv = rope_inv_freq(rotary_dim, theta)
    pos = np.asarray(positions, dtype=np.float32)[:, None]
    ang = (pos * inv[None, :]).astype(np.float32).astype(np.float64)
    return (torch.from_numpy(np.sin(ang).astype(np.float32)),
            torch.from_numpy(np.cos(ang).astype(np.float32)))


def apply_rope(h, sin, cos, rotary_dim):
    """Split-half pairing inside the first R dims: (u, w) = (h[i], h[i+R/2]);
    h[i] = u*cos - w*sin; h[i+R/2] = u*sin + w*cos; the rest passes through
    (applyPreparedRope, model.go:3072-3080).  h: [T, heads, hd]."""
    half = rotary_dim // 2
    if half == 0:
        return h
    s = sin.to(h.dtype)[:, None, :]
    c = cos.to(h.dtype)[:, None, :]
    u, w = h[..., :half], h[..., half:rotary_dim]
    out = h.clone()
    out[..., :half] = u * c - w * s
    out[..., half:rotary_dim] = u * s + w * c
    return out


def attention(q, k, v, window=0):
    """For head h and query position p: scores over keys j = lo..p (the loop bound is
    the causal mask, lo = p-window+1 with a window, model.go:2707-2710), softmax
    with the maximum subtracted, weighted sum of values
    (onlineAttentionWithSink, model.go:3346-3366; weightedVSumEitherWithSink, :3801-3855).
    q: [T, nH, hd] already scaled, k, v: [T, nKV, hd]; query head h reads group
    h // (nH/nKV) (model.go:2828)."""
    T, nH, hd = q.shape
    nKV = k.shape[1]
    rep = nH // nKV
    out = torch.zeros_like(q)
    for h in range(nH):
        g = h // rep
        for p in range(T):
            lo = max(0, p - window + 1) if window > 0 else 0
            s = k[lo:p + 1, g] @ q[p, h]
            w = torch.exp(s - s.max())
            out[p, h] = (w[:, None] * v[lo:p + 1, g]).sum(0) / w.sum()
    return out


def gelu_erf(x):
    """0.5*x*(1+erf(x/sqrt 2)) (geluExact, bert.go:742-744)."""
    return 0.5 * x * (1.0 + torch.erf(x / math.sqrt(2.0)))


def gelu_new(x):
    """x*sigmoid(2*sqrt(2/pi)*(x+0.044715x^3)), the tanh form (geluTanhScalar, fastmath.go:138-141)."""
    return x * torch.sigmoid(1.5957691216057308 * (x + 0.044715 * x * x * x))


ACTIVATIONS = {"gelu": gelu_erf, "gelu_new": gelu_new, "gelu_pytorch_tanh": gelu_new,
               "relu": torch.relu}


def mlp(xn, w1, b1, w2, b2, act):
    """fc2(act(fc1(xn))) with biases, no gate (model.go:2758-2772; forward_batch.go:537-581)."""
    return ACTIVATIONS[act](xn @ w1.T + b1) @ w2.T + b2


def phi_block(x, positions, W, i, cfg):
    """One layer: n = LayerNorm(x); attention branch and MLP branch both read n
    (model.go:2738-2740); x + mlp + attn, the MLP first (model.go:2812-2815).
    Inside attention: bias, optional per-head LayerNorm of q and k, rotation, then
    q * 1/sqrt(hd) (model.go:2677-2706; forward_batch.go:446-469)."""
    nh, nkv, hd, rot = sizes(cfg)
    eps = cfg.get("layer_norm_eps", 1e-5)
    pre = f"model.layers.{i}."
    T = x.shape[0]
    n = layer_norm(x, W[pre + "input_layernorm.weight"], W[pre + "input_layernorm.bias"], eps)
    q = (n @ W[pre + "self_attn.q_proj.weight"].T + W[pre + "self_attn.q_proj.bias"]).reshape(T, nh, hd)
    k = (n @ W[pre + "self_attn.k_proj.weight"].T + W[pre + "self_attn.k_proj.bias"]).reshape(T, nkv, hd)
    v = (n @ W[pre + "self_attn.v_proj.weight"].T + W[pre + "self_attn.v_proj.bias"]).reshape(T, nkv, hd)
    if cfg.get("qk_layernorm", False):
        q = layer_norm(q, W[pre + "self_attn.q_layernorm.weight"], W[pre + "self_attn.q_layernorm.bias"], eps)
        k = layer_norm(k, W[pre + "self_attn.k_layernorm.weight"], W[pre + "self_attn.k_layernorm.bias"], eps)
    sin, cos = rope_tables(positions, rot, cfg.get("rope_theta", 10000.0))
    q = apply_rope(q, sin, cos, rot)
    k = apply_rope(k, sin, cos, rot)
    q = q * (1.0 / math.sqrt(float(hd)))
    a = attention(q, k, v).reshape(T, nh * hd)
    a = a @ W[pre + "self_attn.dense.weight"].T + W[pre + "self_attn.dense.bias"]
    m = mlp(n, W[pre + "mlp.fc1.weight"], W[pre + "mlp.fc1.bias"],
            W[pre + "mlp.fc2.weight"], W[pre + "mlp.fc2.bias"], cfg.get("hidden_act", "gelu_new"))
    return (x + m) + a


def phi_logits(tokens, W, cfg):
    """Logits [T, V] for one whole sequence starting at position 0: embedding, the
    layers, final LayerNorm, output head with bias (model.go:2817, 2555-2564)."""
    x = embedding(tokens, W["model.embed_tokens.weight"])
    positions = list(range(len(tokens)))
    for i in range(cfg["num_hidden_layers"]):
        x = phi_block(x, positions, W, i, cfg)
    eps = cfg.get("layer_norm_eps", 1e-5)
    xn = layer_norm(x, W["model.final_layernorm.weight"], W["model.final_layernorm.bias"], eps)
    head = W["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else W["lm_head.weight"]
    logits = xn @ head.T
    if "lm_head.bias" in W:
        logits = logits + W["lm_head.bias"]
    return logits


# --------------------------------------------------------------------------
# sampling (sampling.go), in float32 like the reference
# --------------------------------------------------------------------------
class Rng:
    """xorshift64 (sampling.go:25-42)."""

    def __init__(self, seed):
        self.state = seed & ((1 << 64) - 1) or 0xDEADBEEFCAFE1337

    def next_f32(self):
        s = self.state
        s ^= (s << 13) & ((1 << 64) - 1)
        s ^= s >> 7
        s ^= (s << 17) & ((1 << 64) - 1)
        self.state = s
        return np.float32(s >> 40) / np.float32(1 << 24)


def _finite(v):
    return np.isfinite(v)


def apply_repeat_penalty(logits, recent, penalty):
    """sampling.go:136-153: once per occurrence in the window."""
    if penalty == 1:
        return
    p = np.float32(penalty)
    for tok in recent:
        if tok < len(logits):
            v = logits[tok]
            if not _finite(v):
                logits[tok] = -np.inf
            elif v > 0:
                logits[tok] = v / p
            else:
                logits[tok] = v * p


def argmax_finite(logits):
    """First index of the maximum, non-finite as -inf (sampling.go:399-418)."""
    v = np.where(np.isfinite(logits), logits, -np.inf)
    return int(np.argmax(v))


def sample(logits, temperature, top_k, top_p, min_p, repeat_penalty, rng, recent):
    """SampleWithScratch (sampling.go:81-130) with sampleTopK (:234-307) and the
    whole-row inverse CDF (:98-129, 156-166)."""
    logits = np.array(logits, dtype=np.float32)
    n = len(logits)
    apply_repeat_penalty(logits, recent, repeat_penalty)
    if temperature < 1e-6:
        return argmax_finite(logits)
    inv_t = np.float32(1.0) / np.float32(temperature)
    if 0 < top_k < n:
        if top_k == 1:
            return argmax_finite(logits)
        v = np.where(np.isfinite(logits), logits, -np.inf).astype(np.float32)
        order = sorted(range(n), key=lambda i: (-v[i], i))[:top_k]
        if v[order[0]] == -np.inf:
            return argmax_finite(logits)
        top = v[order[0]]
        probs = [np.float32(math.exp(float((v[i] - top) * inv_t))) if v[i] > -np.inf else np.float32(0)
                 for i in order]
        s = np.float32(0)
        for p in probs:
            s = np.float32(s + p)
        if s <= 0:
            return order[0]
        cutoff, kept = len(order), s
        if min_p > 0:
            thr = np.float32(min_p) * probs[0]
            acc = np.float32(0)
            for i, p in enumerate(probs):
                if i > 0 and p < thr:
                    cutoff = i
                    break
                acc = np.float32(acc + p)
            s = kept = acc
        if top_p < 1:
            target = np.float32(top_p) * s
            cs = np.float32(0)
            for i in range(cutoff):
                cs = np.float32(cs + probs[i])
                if cs > target:
                    cutoff = i + 1
                    break
            kept = cs
        if kept <= 0:
            return order[0]
        r = np.float32(rng.next_f32() * kept)
        cs = np.float32(0)
        for i in range(cutoff):
            cs = np.float32(cs + probs[i])
            if cs > r:
                return order[i]
        return order[cutoff - 1]
    v = np.where(np.isfinite(logits), logits, -np.inf).astype(np.float32)
    mx = v.max()
    w = np.array([np.float32(math.exp(float((x - mx) * inv_t))) if x > -np.inf else np.float32(0) for x in v],
                 dtype=np.float32)
    total = np.float32(0)
    for x in w:
        total = np.float32(total + x)
    if not (total > 0) or not np.isfinite(total):
        return int(np.argmax(w))
    if top_p < 1 or min_p > 0:
        # sampleTopPFromWeights (sampling.go:171-228)
        thr = np.float32(w.max() * np.float32(1e-5))
        cand = [(i, x) for i, x in enumerate(w) if x >= thr]
        kept_sum = np.float32(0)
        for _, x in cand:
            kept_sum = np.float32(kept_sum + x)
        if kept_sum < np.float32(top_p) * total:
            cand = list(enumerate(w))
        cand.sort(key=lambda t: (-t[1], t[0]))
        cutoff = len(cand)
        if min_p > 0 and cutoff > 0:
            mthr = np.float32(min_p) * cand[0][1]
            total = np.float32(0)
            for i, (_, x) in enumerate(cand):
                if i > 0 and x < mthr:
                    cutoff = i
                    break
                total = np.float32(total + x)
        target = np.float32(top_p) * total
        cs = np.float32(0)
        for i in range(cutoff):
            cs = np.float32(cs + cand[i][1])
            if cs > target:
                cutoff = i + 1
                break
        kept = cs
        if not (kept > 0) or not np.isfinite(kept):
            return int(np.argmax(w))
        r = np.float32(rng.next_f32() * kept)
        cs = np.float32(0)
        for i in range(cutoff):
            cs = np.float32(cs + cand[i][1])
            if cs > r:
                return cand[i][0]
        return cand[cutoff - 1][0]
    r = rng.next_f32()
    cs = np.float32(0)
    for i, x in enumerate(w):
        cs = np.float32(cs + np.float32(x / total))
        if cs > r:
            return i
    return n - 1
