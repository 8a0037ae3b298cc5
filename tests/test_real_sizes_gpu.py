"""The engine at the layer sizes of the published models, against the plain implementation.

Two of the model's layers with everything else as published: Phi-2's sizes (2 of 32 layers: width
2,560, 32 heads of 80 with 32 rotary dims, intermediate 10,240, vocabulary 51,200) and Phi-1.5's (2 of
24 layers: width 2,048, 32 heads of 64, intermediate 8,192).  Random weights written once to a
temporary folder; the plain implementation in 64-bit on the CPU is the oracle.  The reference checks its
own Phi-2 fixture the same way, one token at a time against a batch, within 1e-3 * max(1, |ref|)
(arch_improvements_test.go:129-164, model_families_test.go:440-463, forward_batch_test.go:44-98).
"""
import shutil
import tempfile

import numpy as np
import pytest

import plain_phi
import tiny

pytestmark = pytest.mark.gpu

PHI2_2L = dict(architectures=["PhiForCausalLM"], model_type="phi", num_hidden_layers=2, hidden_size=2560,
               num_attention_heads=32, num_key_value_heads=32, intermediate_size=10240, vocab_size=51200,
               partial_rotary_factor=0.4, rope_theta=10000.0, layer_norm_eps=1e-5, hidden_act="gelu_new",
               qk_layernorm=False, tie_word_embeddings=False, max_position_embeddings=2048,
               initializer_range=0.02, torch_dtype="bfloat16")
PHI15_2L = dict(PHI2_2L, hidden_size=2048, intermediate_size=8192, partial_rotary_factor=0.5)
SIZES = {"phi-2": (PHI2_2L, 2), "phi-1.5": (PHI15_2L, 3)}
TOL = {"float32": 1e-3, "bfloat16": 3e-2}      # times max(1, max |reference|)


class _Case:
    """Folder, plain weights and plain logits of one size, made once and dropped with the module."""

    def __init__(self, label):
        from gopherllm_b200 import write_random_model
        self.cfg, seed = SIZES[label]
        self.folder = tempfile.mkdtemp(prefix=f"gl_{label}_2l_")
        write_random_model(self.folder, dict(self.cfg), seed=seed)
        _, self.W = plain_phi.read_folder(self.folder)
        self._ref = {}
        self._models = {}

    def ref(self, tokens):
        key = tuple(tokens)
        if key not in self._ref:
            self._ref[key] = plain_phi.phi_logits(tokens, self.W, self.cfg).numpy()
        return self._ref[key]

    def model(self, dtype):
        import gopherllm_b200 as gl
        if dtype not in self._models:
            self._models[dtype] = gl.load(self.folder, dtype=dtype, max_tokens=1024)
        return self._models[dtype]

    def drop(self):
        for m in self._models.values():
            m.close()
        self._models.clear()
        self.W = None
        self._ref.clear()
        shutil.rmtree(self.folder, ignore_errors=True)


@pytest.fixture(scope="module", params=sorted(SIZES))
def case(request):
    c = _Case(request.param)
    yield c
    c.drop()


def check(got, ref, dtype, what):
    got = np.asarray(got, dtype=np.float64)
    assert got.shape == ref.shape and np.isfinite(got).all(), what
    scale = max(1.0, np.abs(ref).max())
    for t in range(len(ref)):
        err = np.abs(got[t] - ref[t]).max()
        assert err <= TOL[dtype] * scale, f"{what}: first wrong row {t}: {err:.3e} > {TOL[dtype] * scale:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_last_32_one_by_one(case, dtype):
    V = case.cfg["vocab_size"]
    rng = np.random.default_rng(51)
    toks = tiny.prompt(rng, 200, V)
    ref = case.ref(toks)
    m = case.model(dtype)
    s = m.open_sequence()
    whole = m.step([(s, toks)], [list(range(200))]).cpu().numpy()
    m.close_sequence(s)
    check(whole, ref, dtype, f"{dtype} whole prompt")
    s = m.open_sequence()
    got = [m.step([(s, toks[:168])], [list(range(168))]).cpu().numpy()]
    for t in range(168, 200):
        got.append(m.step([(s, [toks[t]])]).cpu().numpy())
    m.close_sequence(s)
    check(np.concatenate(got), ref, dtype, f"{dtype} last 32 one by one (prompt part ends at 168)")
    m.engine.cache.check()
    m.engine.check_device()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batches_one_after_another(case, dtype):
    """Prompts of unequal lengths in one step, then one token each; shorter requests end earlier and
    the second batch takes their slots and pages."""
    V = case.cfg["vocab_size"]
    rng = np.random.default_rng(52)
    m = case.model(dtype)
    cache = m.engine.cache
    for lens, decs in (([70, 5, 33], [6, 2, 4]), ([3, 65], [5, 3])):
        seqs = [tiny.prompt(rng, a + d, V) for a, d in zip(lens, decs)]
        refs = [case.ref(s) for s in seqs]
        slots = [m.open_sequence() for _ in seqs]
        got = [[] for _ in seqs]
        out = m.step([(slots[i], seqs[i][:lens[i]]) for i in range(len(seqs))],
                     [list(range(n)) for n in lens]).cpu().numpy()
        o = 0
        for i, a in enumerate(lens):
            got[i].append(out[o:o + a])
            o += a
        live = list(range(len(seqs)))
        for step in range(max(decs)):
            live = [i for i in live if step < decs[i]]
            out = m.step([(slots[i], [seqs[i][lens[i] + step]]) for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                if step + 1 == decs[i]:
                    m.close_sequence(slots[i])
        for i in range(len(seqs)):
            check(np.concatenate(got[i]), refs[i], dtype, f"{dtype} batch {lens} request {i} (prompt {lens[i]})")
        cache.check()
        assert cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in cache.groups)
    m.engine.check_device()
