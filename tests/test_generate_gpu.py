"""Generation through the Python entry point and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import plain_phi
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GREEDY = dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0)
_M = {}


def model(name, dtype, max_tokens=2048):
    import gopherllm_b200 as gl
    key = (name, dtype, max_tokens)
    if key not in _M:
        _M[key] = gl.load(tiny.folder(name), dtype=dtype, max_tokens=max_tokens)
    return _M[key]


def plain_greedy(name, prompt, n, stop=()):
    cfg, W = plain_phi.read_folder(tiny.folder(name))
    seq, out = list(prompt), []
    for _ in range(n):
        t = int(plain_phi.phi_logits(seq, W, cfg)[-1].argmax())
        if t in stop:
            return out, "stop"
        out.append(t)
        seq.append(t)
    return out, "length"


@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_equals_plain(name):
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(31)
    prompt = tiny.prompt(rng, 9, cfg["vocab_size"])
    want, _ = plain_greedy(name, prompt, 12)
    m = model(name, "float32")
    got = m.generate(prompt, max_tokens=12, stop_tokens=(), **GREEDY)
    assert got.tokens == want and got.finish_reason == "length"
    assert got.stats.prompt_tokens == 9 and got.stats.generated_tokens == 12
    assert 0 < got.stats.ttft <= got.stats.total_time and got.stats.decode_time > 0
    # bfloat16: every chosen token is the plain argmax given the engine's own prefix, or within rounding of it
    mb = model(name, "bfloat16")
    gb = mb.generate(prompt, max_tokens=12, stop_tokens=(), **GREEDY)
    pcfg, W = plain_phi.read_folder(tiny.folder(name))
    ref = plain_phi.phi_logits(prompt + gb.tokens, W, pcfg).numpy()
    for i, tok in enumerate(gb.tokens):
        row = ref[len(prompt) + i - 1]
        assert row[tok] >= row.max() - 2 * tiny.TOL["bfloat16"] * max(1.0, np.abs(row).max()), i


def test_unequal_prompts_stops_and_batches_one_after_another():
    """Eight requests through a cache that holds three at a time: several batches, slots used
    again; a stop token ends some requests early; each result equals the request run alone."""
    name = "A"
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(32)
    prompts = [tiny.prompt(rng, n, cfg["vocab_size"]) for n in (5, 17, 32, 1, 60, 3, 44, 9)]
    m = model(name, "float32", max_tokens=3 * 128)
    alone = [m.generate(p, max_tokens=20, stop_tokens=(), **GREEDY).tokens for p in prompts]
    # a token that some requests produce within their first 20: generation must stop right before it
    stop = alone[2][7]
    res = m.generate(prompts, max_tokens=20, stop_tokens=(stop,), **GREEDY)
    assert len(res) == len(prompts)
    for r, full in zip(res, alone):
        if stop in full:
            assert r.tokens == full[:full.index(stop)] and r.finish_reason == "stop"
        else:
            assert r.tokens == full and r.finish_reason == "length"
    assert res[2].finish_reason == "stop" and len(res[2].tokens) == alone[2].index(stop) <= 7
    cache = m.engine.cache
    cache.check()
    assert cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in cache.groups)
    # the model's own end-of-sequence id is the default stop token
    eos = cfg["eos_token_id"]
    d = m.generate(prompts[0], max_tokens=20, **GREEDY)
    assert eos not in d.tokens
    # a request that reaches the model's last position ends with "length"
    long = tiny.prompt(rng, 120, cfg["vocab_size"])
    r = m.generate(long, max_tokens=50, stop_tokens=(), **GREEDY)
    assert r.finish_reason == "length" and len(r.tokens) == 128 - 120 + 1
    with pytest.raises(ValueError):
        m.generate(tiny.prompt(rng, 128, cfg["vocab_size"]), max_tokens=5, **GREEDY)
    with pytest.raises(ValueError):
        m.generate([[]], max_tokens=5, **GREEDY)


def test_stop_tokens_in_bfloat16_batches():
    """The bfloat16 engine starts each next step from the sampler's output before the host has seen the
    tokens; a sequence that meets a stop token then has been fed once too often and is dropped, the
    others go on.  Every token of every result must be the plain argmax given the result's own prefix
    (within rounding), a "stop" must come where the stop token is the argmax, and nothing stays held."""
    name = "B"
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(35)
    prompts = [tiny.prompt(rng, n, cfg["vocab_size"]) for n in (7, 21, 2, 40, 13)]
    m = model(name, "bfloat16", max_tokens=5 * 128)
    alone = m.generate(prompts[1], max_tokens=16, stop_tokens=(), **GREEDY).tokens
    stop = alone[5]
    res = m.generate(prompts, max_tokens=16, stop_tokens=(stop,), **GREEDY)
    pcfg, W = plain_phi.read_folder(tiny.folder(name))
    tol = 2 * tiny.TOL["bfloat16"]
    assert any(r.finish_reason == "stop" for r in res) and any(r.finish_reason == "length" for r in res)
    for p, r in zip(prompts, res):
        assert stop not in r.tokens
        ref = plain_phi.phi_logits(p + r.tokens, W, pcfg).numpy()
        for i, tok in enumerate(r.tokens):
            row = ref[len(p) + i - 1]
            assert row[tok] >= row.max() - tol * max(1.0, np.abs(row).max()), i
        if r.finish_reason == "stop":
            row = ref[len(p) + len(r.tokens) - 1]
            assert row[stop] >= row.max() - tol * max(1.0, np.abs(row).max())
        else:
            assert r.finish_reason == "length" and len(r.tokens) == 16
    cache = m.engine.cache
    cache.check()
    assert cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in cache.groups)


def test_sampling_is_seeded_and_independent_of_the_batch():
    name = "B"
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(33)
    a, b, c = (tiny.prompt(rng, n, cfg["vocab_size"]) for n in (12, 40, 3))
    m = model(name, "float32")
    opts = dict(max_tokens=16, temperature=0.9, top_k=30, top_p=0.95, min_p=0.02, repeat_penalty=1.1,
                stop_tokens=())
    r1 = m.generate([a, b], seed=77, **opts)
    r2 = m.generate([a, c], seed=77, **opts)
    r3 = m.generate([a, b], seed=78, **opts)
    assert r1[0].tokens == r2[0].tokens                  # same seed and place: the neighbour does not matter
    assert r1[0].tokens != r3[0].tokens or r1[1].tokens != r3[1].tokens
    assert r1[0].tokens == m.generate(a, seed=77, **opts).tokens
    # the draws follow the reference's sampler: replay them with the plain sampler on plain logits
    pcfg, W = plain_phi.read_folder(tiny.folder(name))
    gen = plain_phi.Rng(77)
    seq, recent = list(a), list(a)[-64:]
    for i, tok in enumerate(r1[0].tokens):
        logits = plain_phi.phi_logits(seq, W, pcfg)[-1].numpy().astype(np.float32)
        want = plain_phi.sample(logits, 0.9, 30, 0.95, 0.02, 1.1, gen, recent)
        assert tok == want, f"draw {i}"
        seq.append(tok)
        recent = (recent + [tok])[-64:]


def test_cancel_between_steps():
    import gopherllm_b200 as gl
    m = model("A", "float32")
    calls = [0]

    def stop():
        calls[0] += 1
        return calls[0] >= 3
    with pytest.raises(gl.GenerationCanceled) as e:
        m.generate([1, 2, 3], max_tokens=50, stop_tokens=(), should_stop=stop, **GREEDY)
    assert e.value.results[0].finish_reason == "canceled" and len(e.value.results[0].tokens) == 3
    m.engine.cache.check()
    assert m.engine.cache.slots.held_count == 0


def test_tokens_are_handed_out_as_they_come():
    """on_token gets (request index, token) for every emitted token, in order per request, the stop
    token never; returning False cancels with what was generated so far."""
    import gopherllm_b200 as gl
    name = "A"
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(36)
    prompts = [tiny.prompt(rng, n, cfg["vocab_size"]) for n in (6, 19, 3)]
    m = model(name, "float32")
    alone = m.generate(prompts[1], max_tokens=10, stop_tokens=(), **GREEDY).tokens
    stop = alone[4]
    seen = {0: [], 1: [], 2: []}
    res = m.generate(prompts, max_tokens=10, stop_tokens=(stop,), on_token=lambda i, t: seen[i].append(t), **GREEDY)
    for i, r in enumerate(res):
        assert seen[i] == r.tokens and stop not in seen[i]
    assert res[1].finish_reason == "stop" and len(res[1].tokens) <= 4
    got = []

    def three(i, t):
        got.append(t)
        return len(got) < 3
    with pytest.raises(gl.GenerationCanceled) as e:
        m.generate(prompts[0], max_tokens=10, stop_tokens=(), on_token=three, **GREEDY)
    assert e.value.results[0].tokens == got and len(got) == 3 and e.value.results[0].finish_reason == "canceled"
    m.engine.cache.check()
    assert m.engine.cache.slots.held_count == 0


def test_command_line():
    folder = tiny.folder("A")
    run = lambda *a: subprocess.run([sys.executable, "-m", "gopherllm_b200", folder, *a], cwd=ROOT,
                                    capture_output=True, text=True, timeout=600)
    want, _ = plain_greedy("A", [5, 17, 3], 6)
    p = run("--prompt", "5 17 3", "--max-tokens", "6", "--temp", "0", "--repeat-penalty", "1", "--dtype", "float32",
            "--stop", "100000")
    assert p.returncode == 0, p.stderr[-2000:]
    assert [int(t) for t in p.stdout.split()] == want and "finish=length" in p.stderr
    p = run("--inspect", "--list-tensors")
    assert p.returncode == 0 and "architecture: PhiForCausalLM (loads as phi)" in p.stdout
    assert "supported: true" in p.stdout and "model.layers.1.mlp.fc2.bias" in p.stdout
    p = run("--bench-json", "--bench-runs", "2", "--max-tokens", "8", "--preset", "deterministic", "--prompt", "1 2 3 4")
    assert p.returncode == 0, p.stderr[-2000:]
    rows = json.loads(p.stdout)
    assert len(rows) == 2 and rows[0]["prompt_tokens"] == 4 and rows[0]["generated_tokens"] <= 8
    assert rows[0]["generated_tokens_per_second"] > 0 and "ttft_ms" in rows[0]
    p = run("--kernel-bench-json", "--kernel-bench-runs", "3")
    assert p.returncode == 0, p.stderr[-2000:]
    kb = json.loads(p.stdout)
    assert kb["format"] == "llm-kernel-bench.v1" and any(k["name"] == "ffn_up" for k in kb["kernels"])
