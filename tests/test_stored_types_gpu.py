"""Folders stored in other types than the compute type load into the serving kernels' types."""
import json
import os
import shutil
import tempfile

import numpy as np
import pytest
import torch

import plain_phi
import tiny

pytestmark = pytest.mark.gpu


def restored(src, stored, label):
    """A copy of folder ``src`` with every tensor stored as ``stored`` (values nudged off the
    bfloat16 grid first) and config.json declaring it."""
    from gopherllm_b200.weights.safetensors_io import TensorFile, index_folder, write_file
    d = tempfile.mkdtemp(prefix=f"gl_{label}_")
    cfg = json.load(open(os.path.join(src, "config.json")))
    cfg["torch_dtype"] = label
    json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
    entries = index_folder(src)
    with TensorFile(entries) as tf:
        tensors = {n: (tf.get(n).float() * 1.003).to(stored) for n in entries}
    write_file(os.path.join(d, "model.safetensors"), tensors.items())
    return d


@pytest.mark.parametrize("stored,label", [(torch.float16, "float16"), (torch.float32, "float32")])
@pytest.mark.parametrize("name", ["A", "C"])
def test_float16_and_float32_folders_reach_the_bfloat16_kernels(name, stored, label):
    """The published Phi checkpoints are float16.  Loaded with dtype="bfloat16" their matrices are
    held in bfloat16, a prompt and a decode step run without the 32-bit CUDA-core product, the log says
    what was rounded, and the logits match the plain implementation fed the rounded weights."""
    import gopherllm_b200 as gl
    from gopherllm_b200 import ops
    cfg = tiny.TINY[name][0]
    d = restored(tiny.folder(name), stored, label)
    said = []
    m = gl.load(d, dtype="bfloat16", max_tokens=512, log=said.append)
    try:
        assert any("rounded to bfloat16" in s and label in s for s in said), said
        blk = m.engine.model.blocks[0]
        assert blk.mixer.w_qkv.dtype == torch.bfloat16 and blk.ffn.w_down.dtype == torch.bfloat16
        assert m.engine.model.embedding.dtype == torch.bfloat16 and blk.mixer.b_qkv.dtype == torch.float32
        rng = np.random.default_rng(61)
        toks = tiny.prompt(rng, 90, cfg["vocab_size"])
        real = ops.gemm_simt

        def no_simt(*a, **k):
            raise AssertionError("a product of the bfloat16 path fell to the 32-bit CUDA-core kernel")
        ops.gemm_simt = no_simt
        try:
            s = m.open_sequence()
            got = [m.step([(s, toks[:80])], [list(range(80))])]
            for t in range(80, 90):
                got.append(m.step([(s, [toks[t]])]))
            m.close_sequence(s)
        finally:
            ops.gemm_simt = real
        got = torch.cat(got).cpu().numpy()
        pcfg, W = plain_phi.read_folder(d, torch.float32)
        W = {n: (t.to(torch.bfloat16) if t.dim() == 2 else t).double() for n, t in W.items()}
        ref = plain_phi.phi_logits(toks, W, pcfg).numpy()
        err, bound = tiny.close(got, ref, "bfloat16")
        assert err <= bound, f"{name} stored as {label}: {err:.3e} > {bound:.3e}"
        # the explicit opt-out keeps them in 32-bit
        k = gl.load(d, dtype="bfloat16", max_tokens=128, keep_stored=True)
        assert k.engine.model.blocks[0].mixer.w_qkv.dtype == torch.float32
        k.close()
    finally:
        m.close()
        shutil.rmtree(d, ignore_errors=True)


def test_a_seed_is_one_tensor_set_in_memory_and_in_a_folder():
    """load_random(config, seed) holds what write_random_model(folder, config, seed) + load(folder)
    holds: the same logits to the bit, in both precisions; with fewer layers, the same first layers."""
    import gopherllm_b200 as gl
    cfg, seed = tiny.TINY["C"]
    rng = np.random.default_rng(62)
    toks = tiny.prompt(rng, 50, cfg["vocab_size"])
    for dtype in ("float32", "bfloat16"):
        a = gl.load(tiny.folder("C"), dtype=dtype, max_tokens=256)
        b = gl.load_random(dict(cfg), seed=seed, dtype=dtype, max_tokens=256)
        outs = []
        for m in (a, b):
            s = m.open_sequence()
            outs.append(m.step([(s, toks)], [list(range(50))]).cpu())
            m.close_sequence(s)
        assert torch.equal(outs[0], outs[1]), dtype
        one = gl.load_random(dict(cfg), seed=seed, dtype=dtype, max_tokens=256, layers=1)
        assert torch.equal(one.engine.model.blocks[0].ffn.w_up, a.engine.model.blocks[0].ffn.w_up)
        assert torch.equal(one.engine.model.head_weight, a.engine.model.head_weight)
        for m in (a, b, one):
            m.close()
