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
