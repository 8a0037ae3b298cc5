"""The plain implementation checked against independent formulas (no device needed)."""
import math

import numpy as np
import torch

import plain_phi
import tiny


def test_parts_against_torch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(7, 33, generator=g, dtype=torch.float64)
    w, b = torch.randn(33, generator=g, dtype=torch.float64), torch.randn(33, generator=g, dtype=torch.float64)
    ref = torch.nn.functional.layer_norm(x, (33,), w, b, 1e-5)
    assert (plain_phi.layer_norm(x, w, b, 1e-5) - ref).abs().max() < 1e-12
    assert (plain_phi.gelu_erf(x) - torch.nn.functional.gelu(x)).abs().max() < 1e-12
    assert (plain_phi.gelu_new(x) - torch.nn.functional.gelu(x, approximate="tanh")).abs().max() < 1e-12
    T, nH, nKV, hd = 9, 4, 2, 8
    q, k, v = (torch.randn(T, n, hd, generator=g, dtype=torch.float64) for n in (nH, nKV, nKV))
    got = plain_phi.attention(q, k, v)
    kk, vv = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
    s = torch.einsum("thd,shd->hts", q, kk)
    s = s.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), -math.inf)
    ref = torch.einsum("hts,shd->thd", torch.softmax(s, -1), vv)
    assert (got - ref).abs().max() < 1e-12
    win = plain_phi.attention(q, k, v, window=3)
    band = torch.tril(torch.ones(T, T, dtype=torch.bool), -3)
    ref = torch.einsum("hts,shd->thd", torch.softmax(s.masked_fill(band, -math.inf), -1), vv)
    assert (win - ref).abs().max() < 1e-12


def test_rope():
    inv = plain_phi.rope_inv_freq(8, 10000.0)
    assert inv.dtype == np.float32 and inv[0] == 1.0 and abs(inv[1] - 0.1) < 1e-7 and abs(inv[3] - 1e-3) < 1e-9
    sin, cos = plain_phi.rope_tables([0, 1, 1000], 8, 10000.0)
    assert sin[0].abs().max() == 0 and (cos[0] == 1).all()
    h = torch.randn(3, 2, 16, dtype=torch.float64)
    r = plain_phi.apply_rope(h, sin, cos, 8)
    assert torch.equal(r[..., 8:], h[..., 8:])                       # partial rotation: the rest passes through
    assert torch.equal(r[0], h[0])                                   # position 0 is the identity
    n0 = (h[..., :8] ** 2).sum(-1)
    assert ((r[..., :8] ** 2).sum(-1) - n0).abs().max() < 1e-6       # a rotation keeps the norm
    # pairs are (i, i + half), not (2i, 2i+1)
    e = torch.zeros(1, 1, 16, dtype=torch.float64)
    e[0, 0, 0] = 1.0
    s1, c1 = plain_phi.rope_tables([1], 8, 10000.0)
    out = plain_phi.apply_rope(e, s1, c1, 8)[0, 0]
    assert abs(out[0] - math.cos(1.0)) < 1e-6 and abs(out[4] - math.sin(1.0)) < 1e-6 and out[1] == 0


def test_whole_model_is_causal_and_dtype_stable():
    cfg, W = plain_phi.read_folder(tiny.folder("A"))
    toks = tiny.prompt(np.random.default_rng(0), 20, cfg["vocab_size"])
    full = plain_phi.phi_logits(toks, W, cfg)
    part = plain_phi.phi_logits(toks[:11], W, cfg)
    assert (full[:11] - part).abs().max() < 1e-10                    # a position does not see later tokens
    cfg32, W32 = plain_phi.read_folder(tiny.folder("A"), dtype=torch.float32)
    f32 = plain_phi.phi_logits(toks, W32, cfg32)
    assert (f32.double() - full).abs().max() < 2e-5


def test_sampler_rules():
    r = plain_phi.Rng(0)
    assert r.state == 0xDEADBEEFCAFE1337
    u = [float(plain_phi.Rng(42).next_f32()) for _ in range(1)]
    assert 0 <= u[0] < 1
    lg = np.array([0.1, 2.0, 2.0, -1.0, np.nan], dtype=np.float32)
    assert plain_phi.sample(lg, 0.0, 0, 1.0, 0.0, 1.0, plain_phi.Rng(1), []) == 1        # first maximum
    assert plain_phi.sample(lg, 0.0, 0, 1.0, 0.0, 2.0, plain_phi.Rng(1), [1]) == 2       # penalty: 2.0/2
    assert plain_phi.sample(lg, 0.0, 0, 1.0, 0.0, 2.0, plain_phi.Rng(1), [1, 2, 2]) == 1  # applied per occurrence
    assert plain_phi.sample(lg, 5.0, 1, 1.0, 0.0, 1.0, plain_phi.Rng(1), []) == 1        # top-k 1 is greedy
    counts = np.zeros(5)
    rng = plain_phi.Rng(7)
    for _ in range(400):
        counts[plain_phi.sample(lg, 1.0, 3, 1.0, 0.0, 1.0, rng, [])] += 1
    assert counts[3] == 0 and counts[4] == 0 and counts[1] > 100 and counts[2] > 100 and counts[0] > 10
    for _ in range(200):                                                                  # min-p drops the tail
        assert plain_phi.sample(lg, 1.0, 4, 1.0, 0.5, 1.0, rng, []) in (1, 2)
    for _ in range(200):                                                                  # nucleus: 0.46 > 0.4
        assert plain_phi.sample(lg, 1.0, 4, 0.4, 0.0, 1.0, rng, []) == 1


def test_golden_outputs_are_unchanged():
    """tests/golden/plain_tiny.json pins the plain implementation and the seeded weights."""
    import json
    import os
    import sys
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, here)
    import make_golden
    now = make_golden.compute()
    with open(os.path.join(here, "plain_tiny.json")) as f:
        then = json.load(f)
    for name in then:
        assert now[name]["tokens"] == then[name]["tokens"]
        assert now[name]["argmax"] == then[name]["argmax"]
        assert np.allclose(now[name]["last_row_first_8"], then[name]["last_row_first_8"], atol=2e-6)
        assert np.allclose(now[name]["row_sums"], then[name]["row_sums"], atol=2e-4)
