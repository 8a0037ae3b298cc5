"""Tiny configurations of the architecture used by the tests, and helpers.

A and B differ in every size and option (layers, width, heads, head size,
intermediate width, vocabulary, rotary share, base, eps, activation, per-head
norm, tied head, positions, weight scale); C adds grouped key/value heads and a
head size that is no power of two.
"""
import os
import tempfile

import numpy as np

TINY_A = dict(architectures=["PhiForCausalLM"], model_type="phi", num_hidden_layers=2, hidden_size=64,
              num_attention_heads=4, num_key_value_heads=4, intermediate_size=256, vocab_size=512,
              partial_rotary_factor=0.5, rope_theta=10000.0, layer_norm_eps=1e-5, hidden_act="gelu_new",
              qk_layernorm=False, tie_word_embeddings=False, max_position_embeddings=128,
              initializer_range=0.02, torch_dtype="bfloat16", eos_token_id=2, bos_token_id=1)
TINY_B = dict(architectures=["PhiForCausalLM"], model_type="phi", num_hidden_layers=3, hidden_size=160,
              num_attention_heads=5, num_key_value_heads=5, intermediate_size=416, vocab_size=1000,
              partial_rotary_factor=0.25, rope_theta=500000.0, layer_norm_eps=1e-6, hidden_act="gelu",
              qk_layernorm=True, tie_word_embeddings=True, max_position_embeddings=256,
              initializer_range=0.05, torch_dtype="bfloat16", eos_token_id=7)
TINY_C = dict(architectures=["PhiForCausalLM"], model_type="phi", num_hidden_layers=2, hidden_size=120,
              num_attention_heads=6, num_key_value_heads=2, head_dim=48, intermediate_size=200,
              vocab_size=777, partial_rotary_factor=0.5, rope_theta=10000.0, layer_norm_eps=1e-5,
              hidden_act="gelu_new", qk_layernorm=True, tie_word_embeddings=False,
              max_position_embeddings=192, initializer_range=0.04, torch_dtype="bfloat16", eos_token_id=3)
TINY = {"A": (TINY_A, 0), "B": (TINY_B, 1), "C": (TINY_C, 5)}

_FOLDERS = {}


def folder(name):
    """A temporary model folder for tiny configuration ``name`` (made once per process)."""
    if name not in _FOLDERS:
        from gopherllm_b200 import write_random_model
        cfg, seed = TINY[name]
        d = tempfile.mkdtemp(prefix=f"gl_tiny_{name}_")
        write_random_model(d, dict(cfg), seed=seed)
        _FOLDERS[name] = d
    return _FOLDERS[name]


def prompt(rng, n, vocab):
    return [int(t) for t in rng.integers(0, vocab, size=n)]


# tolerances: the largest |difference| allowed is tol * max(1, max|reference|)
TOL = {"float32": 1e-4, "bfloat16": 3e-2}


def close(got, ref, dtype):
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all()
    err = np.abs(got - ref).max()
    bound = TOL[dtype] * max(1.0, np.abs(ref).max())
    return err, bound


# --------------------------------------------------------------------------
# a model whose next-token logits hang on one far key and on the positions
# --------------------------------------------------------------------------
FAR_KEY = dict(TINY_A, max_position_embeddings=320, vocab_size=300)
FAR_TOKEN = 7          # the token whose key stands out; prompts hold it once, early
_FAR = {}


def far_key_folder():
    """Tiny configuration A with 320 positions and weights made so that random weights cannot hide a
    wrong rotation, a wrong position or a missed far key.  In layer 0, head 0, one rotary pair (dims
    1 and 5 of 16, angle 0.1 a position): every query has a large bias in dim 1, and the key's row
    for dim 1 points along the normalised embedding of FAR_TOKEN, so wherever that token sits its
    key scores 8*cos(0.1 * distance) while other keys score about 0.  The same token's value in that
    head is large and the output projection is not small, so the residual stream after layer 0, and
    with it the logits, swing with the distance to that one position."""
    if "d" in _FAR:
        return _FAR["d"]
    import json
    import math
    import torch
    from gopherllm_b200 import write_random_model
    import plain_phi
    d = tempfile.mkdtemp(prefix="gl_tiny_far_")
    write_random_model(d, dict(FAR_KEY), seed=9)
    cfg, W = plain_phi.read_folder(d, torch.float32)
    hd, D = 16, FAR_KEY["hidden_size"]
    pre = "model.layers.0."
    n = plain_phi.layer_norm(W["model.embed_tokens.weight"][FAR_TOKEN], W[pre + "input_layernorm.weight"],
                             W[pre + "input_layernorm.bias"], cfg["layer_norm_eps"])
    unit = n / (n * n).sum()
    amp = math.sqrt(8.0 * math.sqrt(hd))               # amp^2 / sqrt(hd) = 8
    W[pre + "self_attn.k_proj.weight"][1] = amp * unit
    W[pre + "self_attn.k_proj.bias"][1] = 0.0
    W[pre + "self_attn.q_proj.weight"][1] = 0.0
    W[pre + "self_attn.q_proj.bias"][1] = amp
    g = torch.Generator().manual_seed(77)
    u = torch.randn(hd, generator=g)
    W[pre + "self_attn.v_proj.weight"][:hd] += 3.0 * u[:, None] * unit[None, :]
    W[pre + "self_attn.dense.weight"][:, :hd] *= 4.0
    from gopherllm_b200.weights.safetensors_io import write_file
    write_file(os.path.join(d, "model.safetensors"), ((k, v.to(torch.bfloat16)) for k, v in sorted(W.items())))
    _FAR["d"] = d
    return d


def far_key_prompt(rng, n, at=3):
    """n tokens without FAR_TOKEN except at position ``at``."""
    toks = [int(t) for t in rng.integers(8, FAR_KEY["vocab_size"], size=n)]
    toks[at] = FAR_TOKEN
    return toks


# A configuration the fused decode layer takes: no per-head norm, a rotary part that is a multiple of
# 16 dims, grouped key/value heads, sizes that are no powers of two.
TINY_D = dict(architectures=["PhiForCausalLM"], model_type="phi", num_hidden_layers=3, hidden_size=168,
              num_attention_heads=6, num_key_value_heads=2, head_dim=64, intermediate_size=200,
              vocab_size=333, partial_rotary_factor=0.5, rope_theta=10000.0, layer_norm_eps=1e-5,
              hidden_act="gelu_new", qk_layernorm=False, tie_word_embeddings=False,
              max_position_embeddings=320, initializer_range=0.05, torch_dtype="bfloat16", eos_token_id=3)
TINY["D"] = (TINY_D, 6)
# six equal layers: enough for a step to repeat the recorded launches of one layer for the later ones
TINY["E"] = (dict(TINY_C, num_hidden_layers=6), 8)
