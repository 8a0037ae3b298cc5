"""Weights: container, checks with one clear error, resident types, random mode (no device needed)."""
import json
import os
import shutil
import tempfile

import pytest
import torch

import plain_phi
import tiny
from gopherllm_b200.api import build_model, write_random_model
from gopherllm_b200.config import load_config
from gopherllm_b200.parts.base import ParamSpec
from gopherllm_b200.weights.loader import (WeightsError, check_folder, load_folder, resident_dtype,
                                           tensor_table)
from gopherllm_b200.weights.safetensors_io import TensorFile, index_folder, read_header, write_file


def table_for(folder):
    arch, cfg = load_config(folder)
    model = build_model(arch, cfg)
    return model, tensor_table(model.parameters(), arch.tensor_names(cfg))


def rewrite(folder, edit):
    """Copy a model folder, letting ``edit`` change the {name: tensor} dict."""
    d = tempfile.mkdtemp(prefix="gl_w_")
    shutil.copy(os.path.join(folder, "config.json"), d)
    entries = index_folder(folder)
    with TensorFile(entries) as tf:
        tensors = {n: tf.get(n).clone() for n in entries}
    edit(tensors)
    write_file(os.path.join(d, "model.safetensors"), tensors.items())
    return d


def test_container_round_trip_and_independent_reader():
    d = tempfile.mkdtemp()
    ts = {"a": torch.arange(6, dtype=torch.float32).reshape(2, 3), "b.c": torch.randn(5).to(torch.bfloat16),
          "i": torch.tensor([1, -2, 3], dtype=torch.int32), "e": torch.zeros(0, 4), "s": torch.tensor(2.5)}
    path = os.path.join(d, "model.safetensors")
    write_file(path, ts.items(), metadata={"k": 1})
    entries, meta = read_header(path)
    assert meta == {"k": "1"} and set(entries) == set(ts)
    with TensorFile(entries) as tf:
        for n, t in ts.items():
            got = tf.get(n)
            assert got.dtype == t.dtype and tuple(got.shape) == tuple(t.shape) and torch.equal(got, t)
    # the package the rest of the world uses reads the same bytes
    from safetensors import safe_open
    with safe_open(path, "pt") as f:
        for n, t in ts.items():
            assert torch.equal(f.get_tensor(n), t)


def test_container_rejects_damage():
    d = tempfile.mkdtemp()
    path = os.path.join(d, "model.safetensors")
    write_file(path, [("a", torch.zeros(4, 4))])
    raw = open(path, "rb").read()
    open(path, "wb").write(raw[:-8])
    with pytest.raises(ValueError, match="exceeds file length"):
        read_header(path)
    open(path, "wb").write(b"\xff" * 4)
    with pytest.raises(ValueError):
        read_header(path)
    with pytest.raises(FileNotFoundError):
        index_folder(tempfile.mkdtemp())


def test_names_follow_the_architecture():
    model, table = table_for(tiny.folder("B"))
    names = set(table)
    assert "model.embed_tokens.weight" in names and "model.final_layernorm.bias" in names
    assert "lm_head.bias" in names and "lm_head.weight" not in names          # tied
    for i in range(3):
        for t in ("input_layernorm.weight", "self_attn.q_proj.weight", "self_attn.k_proj.bias",
                  "self_attn.v_proj.weight", "self_attn.dense.bias", "self_attn.q_layernorm.weight",
                  "self_attn.k_layernorm.bias", "mlp.fc1.weight", "mlp.fc2.bias"):
            assert f"model.layers.{i}.{t}" in names
    _, table_a = table_for(tiny.folder("A"))
    assert "lm_head.weight" in table_a and not any("layernorm.weight" in n and "self_attn" in n for n in table_a)
    check_folder(tiny.folder("A"), table_a)
    # the plain implementation's own reader sees the same tensors
    cfg, W = plain_phi.read_folder(tiny.folder("A"))
    assert set(W) == set(table_a)


def test_one_error_lists_missing_unexpected_and_wrong_shapes():
    src = tiny.folder("A")
    _, table = table_for(src)

    def edit(t):
        del t["model.layers.1.mlp.fc2.bias"]
        del t["lm_head.weight"]
        t["model.layers.0.self_attn.rotary_emb.inv_freq"] = torch.zeros(4)
        t["model.layers.0.mlp.fc1.weight"] = torch.zeros(255, 64, dtype=torch.bfloat16)
        t["model.final_layernorm.weight"] = torch.zeros(64, dtype=torch.int32)
    bad = rewrite(src, edit)
    with pytest.raises(WeightsError) as e:
        check_folder(bad, table)
    msg = str(e.value)
    assert e.value.missing == ["lm_head.weight", "model.layers.1.mlp.fc2.bias"]
    assert e.value.unexpected == ["model.layers.0.self_attn.rotary_emb.inv_freq"]
    assert len(e.value.wrong) == 2
    for needle in ("missing tensors (2)", "unexpected tensors (1)", "wrong shapes or types (2)",
                   "model.layers.0.mlp.fc1.weight is [255, 64], the model wants [256, 64]", "stored as I32"):
        assert needle in msg, needle


def test_tied_head_may_lack_its_bias_and_carry_a_copy():
    src = tiny.folder("B")
    _, table = table_for(src)

    def edit(t):
        del t["lm_head.bias"]
        t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    d = rewrite(src, edit)
    with pytest.raises(WeightsError):
        check_folder(d, table)                                  # the copy is unexpected unless told
    check_folder(d, table, ignore=("lm_head.weight",))
    tensors, _ = load_folder(d, table, torch.float32, "cpu", ignore=("lm_head.weight",))
    assert torch.count_nonzero(tensors["head/bias"]) == 0


def test_fused_projections_are_taken_in_place_of_split_ones():
    """A file with the three projections of a layer as one matrix and one bias (rows Q, K, V) loads to
    the same tensors as the split file; a fused tensor with the wrong number of rows is one clear line."""
    src = tiny.folder("B")                                        # grouped heads: q, k and v differ in rows
    arch, cfg = load_config(src)
    model, table = table_for(src)
    fused = arch.tensor_names(cfg).fused()
    want, _ = load_folder(src, table, torch.float32, "cpu")

    def fuse(t, layers, drop_rows=0):
        for i in layers:
            base = f"model.layers.{i}.self_attn."
            for suffix in ("weight", "bias"):
                parts = [t.pop(f"{base}{p}_proj.{suffix}") for p in ("q", "k", "v")]
                whole = torch.cat(parts, dim=0)
                t[f"{base}Wqkv.{suffix}"] = whole[:whole.shape[0] - drop_rows].contiguous()
    n_layers = cfg.num_hidden_layers
    d = rewrite(src, lambda t: fuse(t, range(n_layers)))
    with pytest.raises(WeightsError):
        check_folder(d, table)                                    # not told about fused tensors: unknown names
    got, _ = load_folder(d, table, torch.float32, "cpu", fused=fused)
    assert set(got) == set(want) and all(torch.equal(got[k], want[k]) for k in want)
    d = rewrite(src, lambda t: fuse(t, [0]))                      # one layer fused, the others split
    got, _ = load_folder(d, table, torch.float32, "cpu", fused=fused)
    assert all(torch.equal(got[k], want[k]) for k in want)
    d = rewrite(src, lambda t: fuse(t, [1], drop_rows=1))
    with pytest.raises(WeightsError) as e:
        check_folder(d, table, fused=fused)
    assert not e.value.missing and not e.value.unexpected and len(e.value.wrong) == 2
    assert "model.layers.1.self_attn.Wqkv.weight is [" in str(e.value) and "the rows of" in str(e.value)


def test_resident_types():
    m, v, i = ParamSpec((2, 2)), ParamSpec((2,), "vector"), ParamSpec((2,), "table_int")
    bf, f32, f16, f64 = torch.bfloat16, torch.float32, torch.float16, torch.float64
    assert resident_dtype(m, bf, bf) == bf            # kept in bfloat16
    assert resident_dtype(m, f16, bf) == bf           # float16 (the published checkpoints) is rounded to bfloat16
    assert resident_dtype(m, f16, bf, f16) == bf
    assert resident_dtype(m, f32, bf) == bf           # a checkpoint that declares nothing: brought to the compute type
    assert resident_dtype(m, f32, bf, f32) == bf      # a 32-bit checkpoint as a whole is rounded
    assert resident_dtype(m, f64, bf, f32) == bf
    assert resident_dtype(m, f32, bf, bf) == f32      # stored in 32-bit inside a 16-bit checkpoint: stays so
    assert resident_dtype(m, f32, bf, f16) == f32
    assert resident_dtype(m, f16, bf, f16, keep_stored=True) == f32     # the explicit opt-out: exact and slow
    assert resident_dtype(m, f32, bf, bf, keep_stored=False) == bf
    assert resident_dtype(m, bf, f32) == f32          # the 32-bit path widens everything
    assert resident_dtype(m, f16, f32) == f32
    assert resident_dtype(v, bf, bf) == f32
    assert resident_dtype(v, f16, bf, f16) == f32
    assert resident_dtype(i, torch.int64, bf) == torch.int32
    src = tiny.folder("A")

    def edit(t):
        t["model.layers.0.mlp.fc1.weight"] = t["model.layers.0.mlp.fc1.weight"].float()
    d = rewrite(src, edit)
    _, table = table_for(d)
    got, nbytes = load_folder(d, table, bf, "cpu", declared=bf)
    assert got["layers/0/ffn/up.weight"].dtype == f32 and got["layers/1/ffn/up.weight"].dtype == bf
    assert got["layers/0/norm/weight"].dtype == f32 and got["embedding"].dtype == bf and nbytes > 0


def test_other_stored_types_are_rounded_to_the_compute_type():
    """A folder stored as float16, and one stored as float32 as a whole, load into bfloat16 matrices
    that equal the stored values rounded to nearest even; the log says that it happened."""
    src = tiny.folder("A")
    _, W = plain_phi.read_folder(src, torch.float32)
    for stored, label in ((torch.float16, "float16"), (torch.float32, "float32")):
        def edit(t):
            for n in t:
                t[n] = (t[n].float() * 1.003).to(stored)       # values that are not bfloat16 numbers already
        d = rewrite(src, edit)
        cfg = json.load(open(os.path.join(d, "config.json")))
        cfg["torch_dtype"] = label
        json.dump(cfg, open(os.path.join(d, "config.json"), "w"))
        _, table = table_for(d)
        said = []
        got, _ = load_folder(d, table, torch.bfloat16, "cpu", progress=said.append, declared=stored)
        w = got["layers/1/mixer/q.weight"]
        assert w.dtype == torch.bfloat16 and got["layers/1/mixer/q.bias"].dtype == torch.float32
        want = (W["model.layers.1.self_attn.q_proj.weight"] * 1.003).to(stored).to(torch.bfloat16)
        assert torch.equal(w, want)
        assert any("rounded to bfloat16" in line and label in line for line in said), said
        kept, _ = load_folder(d, table, torch.bfloat16, "cpu", declared=stored, keep_stored=True)
        assert kept["layers/1/mixer/q.weight"].dtype == torch.float32
        wide, _ = load_folder(d, table, torch.float32, "cpu", declared=stored)
        assert all(t.dtype == torch.float32 for t in wide.values())


def test_random_mode_is_seeded_and_shaped():
    cfg = dict(tiny.TINY_A)
    a, b, c = tempfile.mkdtemp(), tempfile.mkdtemp(), tempfile.mkdtemp()
    write_random_model(a, cfg, seed=3)
    write_random_model(b, cfg, seed=3)
    write_random_model(c, cfg, seed=4)
    assert json.load(open(os.path.join(a, "config.json")))["hidden_size"] == 64
    _, Wa = plain_phi.read_folder(a)
    _, Wb = plain_phi.read_folder(b)
    _, Wc = plain_phi.read_folder(c)
    assert all(torch.equal(Wa[n], Wb[n]) for n in Wa)
    assert not torch.equal(Wa["lm_head.weight"], Wc["lm_head.weight"])
    w = Wa["model.layers.0.mlp.fc1.weight"]
    assert abs(w.std().item() - 0.02) < 0.002 and abs(w.mean().item()) < 0.002
    # drawn several tensors at a time or one by one, in a folder or in memory: one seed is one tensor set
    from gopherllm_b200.weights.loader import random_tensors
    _, table = table_for(a)
    one = dict(random_tensors(table, 3, 0.02, torch.bfloat16, workers=0))
    many = dict(random_tensors(table, 3, 0.02, torch.bfloat16, workers=4))
    assert list(one) == list(many) == sorted(table)
    assert all(torch.equal(one[n], many[n]) and torch.equal(one[n].double(), Wa[n]) for n in one)
    g = Wa["model.layers.1.input_layernorm.weight"]
    assert abs(g.mean().item() - 1.0) < 0.02 and 0.005 < g.std().item() < 0.04
    assert 0.005 < Wa["model.layers.1.self_attn.dense.bias"].std().item() < 0.04
    cfg_b = dict(tiny.TINY_B)
    d = tempfile.mkdtemp()
    write_random_model(d, cfg_b, seed=1)
    _, Wd = plain_phi.read_folder(d)
    assert abs(Wd["model.layers.0.mlp.fc1.weight"].std().item() - 0.05) < 0.004      # initializer_range
    model, table = table_for(d)
    check_folder(d, table)


def test_deeper_parameter_keys_reach_the_names_or_are_refused():
    """A part nested inside a slot's part declares "sub/weight": the tensor table hands the names
    "sub.weight" (not a truncated key); a key no rule covers is an error."""
    from gopherllm_b200.parts import ParamSpec
    from gopherllm_b200.weights.loader import tensor_table

    class Names:
        embedding, final_norm, head = "e", "fn", "hd"

        def layer(self, i, slot, key):
            return f"L{i}.{slot}.{key}"
    t = tensor_table({"embedding": ParamSpec((4, 2)), "layers/3/mixer/inner/gate/weight": ParamSpec((2, 2)),
                      "final_norm/weight": ParamSpec((2,), "vector")}, Names())
    assert set(t) == {"e", "L3.mixer.inner.gate.weight", "fn.weight"}
    with pytest.raises(KeyError):
        tensor_table({"layers/3/mixer": ParamSpec((2, 2))}, Names())
    with pytest.raises(KeyError):
        tensor_table({"positions": ParamSpec((2, 2))}, Names())       # a position table without a name for it
