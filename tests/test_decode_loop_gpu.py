"""The on-device decode loop (the path the device-timed benchmark figure comes from) against the
generation loop and the plain implementation, and steps whose logits hang on positions and on one far key."""
import numpy as np
import pytest
import torch

import plain_phi
import tiny

pytestmark = pytest.mark.gpu
GREEDY = dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0)
SAMPLED = dict(temperature=0.9, top_k=50, top_p=0.95, min_p=0.0, repeat_penalty=1.1)
_M = {}


def model(folder, dtype, max_tokens=2048):
    import gopherllm_b200 as gl
    key = (folder, dtype, max_tokens)
    if key not in _M:
        _M[key] = gl.load(folder, dtype=dtype, max_tokens=max_tokens)
    return _M[key]


def loop_tokens(m, prompts, steps, options, seed):
    """Prompts in one step, the first token sampled from their logits, then ``steps - 1`` more tokens
    from Engine.decode_loop: what Model.generate does, with the loop on the device."""
    from gopherllm_b200.sampling.sampler import DeviceSampler, SamplerConfig, request_seed
    eng = m.engine
    sampler = DeviceSampler(SamplerConfig(**options), [request_seed(seed, i) for i in range(len(prompts))],
                            prompts, m.spec.vocab, eng.device)
    slots = [eng.open() for _ in prompts]
    logits = eng.step([(s, p) for s, p in zip(slots, prompts)])
    first = sampler.sample(logits).tolist()
    out = [[t] for t in first]
    # two calls, so that the second starts a captured step from other positions than it was captured at
    cut = max(1, (steps - 1) // 3)
    fed = first
    for n in (cut, steps - 1 - cut):
        if n < 1:
            continue
        hist = eng.decode_loop(slots, fed, n, sampler).cpu().tolist()
        for row in hist:
            for i, t in enumerate(row):
                out[i].append(t)
        fed = hist[-1]
    lens = [eng.cache.length(s) for s in slots]
    for s in slots:
        eng.close(s)
    return out, lens


@pytest.mark.parametrize("options", [GREEDY, SAMPLED], ids=["greedy", "sampled"])
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_decode_loop_equals_generate(name, dtype, options):
    """At least 40 steps across a page's edge, from prompts of unequal lengths: the loop's tokens are
    the generation loop's for the same prompts and seeds, and the cache holds what was fed."""
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(41)
    prompts = [tiny.prompt(rng, n, cfg["vocab_size"]) for n in (40, 9, 63)]
    steps = 44
    m = model(tiny.folder(name), dtype)
    want = m.generate(prompts, max_tokens=steps, stop_tokens=(), seed=11, **options)
    got, lens = loop_tokens(m, prompts, steps, options, seed=11)
    for i, (g, w) in enumerate(zip(got, want)):
        assert g == w.tokens, f"{name} {dtype}: request {i} differs first at token " \
                              f"{next(k for k, (a, b) in enumerate(zip(g, w.tokens)) if a != b)}"
    assert lens == [len(p) + steps - 1 for p in prompts]       # the last token was chosen, not fed
    m.engine.cache.check()
    assert m.engine.cache.slots.held_count == 0
    m.engine.check_device()


def _far_model(dtype):
    return model(tiny.far_key_folder(), dtype, max_tokens=4 * 320)


def _far_plain(tokens):
    key = ("far", tuple(tokens))
    if key not in _M:
        cfg, W = plain_phi.read_folder(tiny.far_key_folder())
        _M[key] = plain_phi.phi_logits(tokens, W, cfg).numpy()
    return _M[key]


def test_far_key_model_is_sensitive():
    """The made-up weights do what they are for: without the far token, or with every query rotated as
    at one fixed position, the plain logits move by many times the tolerance of the tests below."""
    rng = np.random.default_rng(42)
    toks = tiny.far_key_prompt(rng, 200)
    ref = _far_plain(toks)
    bound = tiny.TOL["bfloat16"] * max(1.0, np.abs(ref).max())
    other = list(toks)
    other[3] = 9
    moved = np.abs(_far_plain(other) - ref).max(axis=1)
    assert (moved[100:] > 3 * bound).mean() > 0.5 and moved.max() > 15 * bound


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_key_whole_then_token_by_token(dtype):
    """A prompt of 70 tokens, then 130 single-token steps (the bfloat16 ones replayed from captured
    graphs, with rotation and cache write inside decode attention): every position's logits against
    the plain implementation; and two steps' logits held by the caller stay what they were."""
    rng = np.random.default_rng(43)
    toks = tiny.far_key_prompt(rng, 200)
    ref = _far_plain(toks)
    m = _far_model(dtype)
    s = m.open_sequence()
    got = [m.step([(s, toks[:70])], [list(range(70))])]
    for t in range(70, 200):
        got.append(m.step([(s, [toks[t]])]))
    m.close_sequence(s)
    assert got[-1].data_ptr() != got[-2].data_ptr()
    assert not torch.equal(got[-1], got[-2]), "two steps' logits are the same tensor contents"
    got = torch.cat(got).cpu().numpy()
    for t in range(200):
        err, bound = tiny.close(got[t], ref[t], dtype)
        assert err <= bound, f"{dtype}: first wrong position {t}: {err:.3e} > {bound:.3e}"
    m.engine.check_device()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_far_key_through_the_decode_loop(dtype):
    """Greedy tokens of the on-device loop, 150 steps from a prompt of 100: each is the plain
    implementation's argmax given the loop's own prefix (within rounding), and they are the
    generation loop's tokens."""
    rng = np.random.default_rng(44)
    prompts = [tiny.far_key_prompt(rng, 100), tiny.far_key_prompt(rng, 37, at=30)]
    m = _far_model(dtype)
    steps = 150
    got, _ = loop_tokens(m, prompts, steps, GREEDY, seed=3)
    want = m.generate(prompts, max_tokens=steps, stop_tokens=(), seed=3, **GREEDY)
    for p, g, w in zip(prompts, got, want):
        ref = _far_plain(p + g)
        tol = (1e-3 if dtype == "float32" else 2 * tiny.TOL["bfloat16"]) * max(1.0, np.abs(ref).max())
        for i, tok in enumerate(g):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - tol, f"{dtype}: token {i} is not the plain argmax ({row.max() - row[tok]:.3e})"
        assert g == w.tokens
    m.engine.cache.check()


def test_a_step_that_fails_midway_leaves_the_cache_sound():
    """The model's forward raises after the step's pages were reserved: the sequence keeps its length,
    no page is lost or owned twice, the same step can be run again, and closing gives everything back."""
    m = model(tiny.folder("A"), "float32")
    eng, cache = m.engine, m.engine.cache
    rng = np.random.default_rng(45)
    toks = tiny.prompt(rng, 100, tiny.TINY_A["vocab_size"])
    s = m.open_sequence()
    m.step([(s, toks[:10])])
    real = eng.model.forward

    def broken(ctx, c):
        raise RuntimeError("made to fail")
    eng.model.forward = broken
    try:
        with pytest.raises(RuntimeError, match="made to fail"):
            m.step([(s, toks[10:90])])
    finally:
        eng.model.forward = real
    assert cache.length(s) == 10
    cache.check()
    got = m.step([(s, toks[10:90])]).cpu().numpy()
    cfg, W = plain_phi.read_folder(tiny.folder("A"))
    ref = plain_phi.phi_logits(toks[:90], W, cfg)[-1].numpy()
    err, bound = tiny.close(got[0], ref, "float32")
    assert err <= bound
    m.close_sequence(s)
    cache.check()
    assert cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in cache.groups)
