"""Layers that see a window of the last w positions beside layers that see every position.

A toy architecture registered from here (Phi's parallel block; every second layer's attention sees the
last ``window`` positions only): nothing inside gopherllm_b200 is edited, and it is nobody's model.
Its layers ask the cache for two kinds of storage, so the cache makes two groups; the group with the
window gives a sequence's pages back once they lie before every window still to come.  Checked here:
the logits of prompts in pieces and of single-token steps against the same model written out plainly
in 64-bit (the window's edge moves over a page's edge on the way), and the pages the cache holds."""
import dataclasses
import math
import tempfile

import numpy as np
import pytest
import torch

import plain_phi
import tiny

pytestmark = pytest.mark.gpu
WINDOW = 70
CFG = dict(tiny.TINY_A, architectures=["ToyWindowForCausalLM"], model_type="toy-window", num_hidden_layers=4,
           max_position_embeddings=320, window=WINDOW)


def define_toy_window():
    from gopherllm_b200.config.phi import PhiConfig, PhiTensorNames, phi_model_spec
    from gopherllm_b200.config.registry import Architecture, register_architecture, resolve_architecture

    if resolve_architecture("toy-window") is None:
        class WindowConfig:
            def __init__(self, phi, window):
                self.phi, self.window = phi, window

            @classmethod
            def from_dict(cls, d):
                return cls(PhiConfig.from_dict({k: v for k, v in d.items() if k != "window"}), int(d["window"]))

            def to_dict(self):
                d = self.phi.to_dict()
                d.update(architectures=["ToyWindowForCausalLM"], model_type="toy-window", window=self.window)
                return d

            def __getattr__(self, k):
                return getattr(self.phi, k)

        def spec_of(c):
            spec = phi_model_spec(c.phi)
            layers = tuple(dataclasses.replace(b, mixer=dataclasses.replace(b.mixer, window=c.window if i % 2 else 0))
                           for i, b in enumerate(spec.layers))
            return dataclasses.replace(spec, layers=layers)

        register_architecture(Architecture("toy-window", WindowConfig, spec_of, lambda c: PhiTensorNames(c.phi)),
                              aliases=["ToyWindow"])
    return resolve_architecture("toy-window")


def plain_logits(tokens, W, cfg):
    """plain_phi.phi_logits with a window on every second layer (the block of plain_phi.phi_block, its
    attention given the window)."""
    nh, nkv, hd, rot = plain_phi.sizes(cfg)
    eps = cfg.get("layer_norm_eps", 1e-5)
    x = plain_phi.embedding(tokens, W["model.embed_tokens.weight"])
    T = len(tokens)
    sin, cos = plain_phi.rope_tables(list(range(T)), rot, cfg.get("rope_theta", 10000.0))
    for i in range(cfg["num_hidden_layers"]):
        pre = f"model.layers.{i}."
        n = plain_phi.layer_norm(x, W[pre + "input_layernorm.weight"], W[pre + "input_layernorm.bias"], eps)
        q = (n @ W[pre + "self_attn.q_proj.weight"].T + W[pre + "self_attn.q_proj.bias"]).reshape(T, nh, hd)
        k = (n @ W[pre + "self_attn.k_proj.weight"].T + W[pre + "self_attn.k_proj.bias"]).reshape(T, nkv, hd)
        v = (n @ W[pre + "self_attn.v_proj.weight"].T + W[pre + "self_attn.v_proj.bias"]).reshape(T, nkv, hd)
        q = plain_phi.apply_rope(q, sin, cos, rot) * (1.0 / math.sqrt(float(hd)))
        k = plain_phi.apply_rope(k, sin, cos, rot)
        a = plain_phi.attention(q, k, v, window=cfg["window"] if i % 2 else 0).reshape(T, nh * hd)
        a = a @ W[pre + "self_attn.dense.weight"].T + W[pre + "self_attn.dense.bias"]
        m = plain_phi.mlp(n, W[pre + "mlp.fc1.weight"], W[pre + "mlp.fc1.bias"], W[pre + "mlp.fc2.weight"],
                          W[pre + "mlp.fc2.bias"], cfg.get("hidden_act", "gelu_new"))
        x = (x + m) + a
    xn = plain_phi.layer_norm(x, W["model.final_layernorm.weight"], W["model.final_layernorm.bias"], eps)
    return xn @ W["lm_head.weight"].T + W["lm_head.bias"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windowed_layers_beside_full_ones(dtype):
    import gopherllm_b200 as gl
    define_toy_window()
    folder = tempfile.mkdtemp(prefix="gl_toy_window_")
    gl.write_random_model(folder, dict(CFG), seed=4)
    cfg, W = plain_phi.read_folder(folder)
    m = gl.load(folder, dtype=dtype, max_tokens=3 * 320)
    assert m.architecture.name == "toy-window"
    cache = m.engine.cache
    assert len(cache.groups) == 2 and sorted(g.req.window for g in cache.groups) == [0, WINDOW]
    windowed = next(g for g in cache.groups if g.req.window)
    full = next(g for g in cache.groups if not g.req.window)
    rng = np.random.default_rng(5)
    V = CFG["vocab_size"]
    seqs = [tiny.prompt(rng, n, V) for n in (300, 150)]
    refs = [plain_logits(s, W, cfg).numpy() for s in seqs]
    slots = [m.open_sequence() for _ in seqs]
    # the prompts in pieces of unequal sizes, every position wanted, then single tokens; the short one ends earlier
    done = [0, 0]
    for piece in ((100, 40), (31, 64), (90, 20)):
        runs = [(slots[i], seqs[i][done[i]:done[i] + piece[i]]) for i in range(2)]
        out = m.step(runs, [list(range(p)) for p in piece]).cpu().numpy()
        row = 0
        for i in range(2):
            err, bound = tiny.close(out[row:row + piece[i]], refs[i][done[i]:done[i] + piece[i]], dtype)
            assert err <= bound, (i, done[i], err, bound)
            row += piece[i]
            done[i] += piece[i]
        cache.check()
        for i in range(2):                              # the windowed group holds the pages from the window's start on
            held = sum(1 for p in cache._pages[slots[i]][windowed.gid] if p >= 0)
            first = max(0, done[i] - WINDOW + 1) // 64
            assert held == -(-done[i] // 64) - first, (i, done[i], held)
            assert sum(1 for p in cache._pages[slots[i]][full.gid] if p >= 0) == -(-done[i] // 64)
    for step in range(26):
        live = [i for i in range(2) if done[i] < len(seqs[i])]
        out = m.step([(slots[i], [seqs[i][done[i]]]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            err, bound = tiny.close(out[r], refs[i][done[i]], dtype)
            assert err <= bound, (i, done[i], err, bound)
            done[i] += 1
            if done[i] == len(seqs[i]):
                m.close_sequence(slots[i])
        cache.check()
    assert done[1] == 150 and done[0] == 247
    # a sequence of 247 positions: four pages in the group that sees everything, two where the window is 70
    assert sum(1 for p in cache._pages[slots[0]][full.gid] if p >= 0) == 4
    assert sum(1 for p in cache._pages[slots[0]][windowed.gid] if p >= 0) == 2
    m.close_sequence(slots[0])
    cache.check()
    assert all(g.pool.held_count == 0 for g in cache.groups)
    m.engine.check_device()
    m.close()
