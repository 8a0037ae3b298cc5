"""bin/trace_run as a user runs it: a subprocess fed JSON steps on standard input."""
import json
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

import plain_phi
import tiny

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def build_trace(cfg, rng):
    """Steps and, for every step that wants logits, the (request, positions) they belong to."""
    V, P = cfg["vocab_size"], cfg["max_position_embeddings"]
    steps, expect, seqs = [], {}, {}
    n = [0]

    def add(entries, end=()):
        i = n[0]
        n[0] += 1
        steps.append({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w, _ in entries],
                      "end": list(end)})
        wanted = [(r, p0 + k) for r, t, w, p0 in entries for k in w]
        if wanted:
            expect[i] = wanted

    # 1. a request alone and whole, logits everywhere
    seqs["whole"] = tiny.prompt(rng, P - 1, V)
    add([("whole", seqs["whole"], list(range(P - 1)), 0)], end=["whole"])
    # 2. all but the last 32 tokens in one step, then one by one
    seqs["tail"] = tiny.prompt(rng, 100, V)
    add([("tail", seqs["tail"][:68], list(range(68)), 0)])
    for t in range(68, 100):
        add([("tail", [seqs["tail"][t]], [0], t)], end=["tail"] if t == 99 else [])
    # 3. two batches of unequal lengths, one after the other; shorter requests end earlier
    for bi, (lens, decs) in enumerate([([70, 3, 64], [12, 2, 5]), ([1, 129, 20, 7], [9, 3, 1, 6])]):
        ids = [f"b{bi}r{k}" for k in range(len(lens))]
        for r, a, d in zip(ids, lens, decs):
            seqs[r] = tiny.prompt(rng, a + d, V)
        add([(r, seqs[r][:a], [a - 1], 0) for r, a in zip(ids, lens)])
        for s in range(max(decs)):
            live = [(r, a, d) for r, a, d in zip(ids, lens, decs) if s < d]
            add([(r, [seqs[r][a + s]], [0], a + s) for r, a, d in live],
                end=[r for r, a, d in live if s + 1 == d])
    # a step that wants nothing writes no file
    seqs["quiet"] = tiny.prompt(rng, 5, V)
    add([("quiet", seqs["quiet"], [], 0)], end=["quiet"])
    return steps, expect, seqs


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(dtype):
    name = "B"
    cfg = tiny.TINY[name][0]
    folder = tiny.folder(name)
    steps, expect, seqs = build_trace(cfg, np.random.default_rng(21))
    out = tempfile.mkdtemp(prefix="gl_trace_")
    # most tokens live at once: 4 requests of the second batch, each rounded up to 64
    max_tokens = 64 + 192 + 64 + 64
    env = dict(os.environ)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", dtype, "--out", out, "--max-tokens", str(max_tokens)],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                          text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    done = [line for line in proc.stdout.splitlines() if line.startswith("done ")]
    assert done == [f"done {s['step']}" for s in steps]
    pcfg, W = plain_phi.read_folder(folder)
    ref = {r: plain_phi.phi_logits(t, W, pcfg).numpy() for r, t in seqs.items()}
    V = cfg["vocab_size"]
    for s in steps:
        path = os.path.join(out, f"{s['step']}.f32")
        if s["step"] not in expect:
            assert not os.path.exists(path)
            continue
        got = np.fromfile(path, dtype="<f4").reshape(-1, V)
        want = np.stack([ref[r][p] for r, p in expect[s["step"]]])
        err, bound = tiny.close(got, want, dtype)
        assert err <= bound, f"{dtype} step {s['step']} ({expect[s['step']][:3]}…): {err:.3e} > {bound:.3e}"


def test_trace_run_refuses_more_tokens_than_the_cache_holds():
    folder = tiny.folder("A")
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1] * 65, "want": [0]}], "end": []}]
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                           "--dtype", "float32", "--out", tempfile.mkdtemp(), "--max-tokens", "64"],
                          input=json.dumps(steps[0]) + "\n", capture_output=True, text=True, timeout=600)
    assert proc.returncode != 0 and "pages" in proc.stderr
