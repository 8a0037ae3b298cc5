"""The engine against the plain implementation: every way of cutting the work."""
import numpy as np
import pytest
import torch

import plain_phi
import tiny

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
_PLAIN = {}
_MODELS = {}


def plain_logits(name, tokens):
    key = (name, tuple(tokens))
    if key not in _PLAIN:
        cfg, W = plain_phi.read_folder(tiny.folder(name))
        _PLAIN[key] = plain_phi.phi_logits(tokens, W, cfg).numpy()
    return _PLAIN[key]


def model(name, dtype):
    import gopherllm_b200 as gl
    key = (name, dtype)
    if key not in _MODELS:
        _MODELS[key] = gl.load(tiny.folder(name), dtype=dtype, max_tokens=1024)
    return _MODELS[key]


def check(got, ref, dtype, what):
    err, bound = tiny.close(got, ref, dtype)
    assert err <= bound, f"{what}: max |diff| {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompt_every_position(name, dtype):
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(10)
    m = model(name, dtype)
    for n in (1, 7, 64, 65, cfg["max_position_embeddings"] - 1):
        toks = tiny.prompt(rng, n, cfg["vocab_size"])
        s = m.open_sequence()
        got = m.step([(s, toks)], [list(range(n))]).cpu().numpy()
        m.close_sequence(s)
        check(got, plain_logits(name, toks), dtype, f"{name} whole n={n}")
    m.engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_last_32_tokens_one_by_one(name, dtype):
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(11)
    m = model(name, dtype)
    n = cfg["max_position_embeddings"] - 3
    toks = tiny.prompt(rng, n, cfg["vocab_size"])
    ref = plain_logits(name, toks)
    s = m.open_sequence()
    head = n - 32
    got = [m.step([(s, toks[:head])], [list(range(head))]).cpu().numpy()]
    for t in range(head, n):
        got.append(m.step([(s, [toks[t]])], [[0]]).cpu().numpy())
    m.close_sequence(s)
    got = np.concatenate(got)
    for t in range(n):      # find the first wrong place, not just the largest error
        err, bound = tiny.close(got[t], ref[t], dtype)
        assert err <= bound, f"{name} {dtype}: first wrong position {t} (prompt part ends at {head}): {err:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_first_tokens_of_a_sequence(name, dtype):
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(12)
    m = model(name, dtype)
    toks = tiny.prompt(rng, 6, cfg["vocab_size"])
    ref = plain_logits(name, toks)
    s = m.open_sequence()
    for t in range(6):      # from the very first token, one at a time
        got = m.step([(s, [toks[t]])], [[0]]).cpu().numpy()
        check(got[0], ref[t], dtype, f"{name} position {t} decoded from an empty cache")
    m.close_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_unequal_batches_one_after_another(name, dtype):
    """Prompts of unequal lengths in one step, then one token each; shorter requests end
    earlier; a second batch reuses the slots and pages, one slot after a longer sequence."""
    cfg = tiny.TINY[name][0]
    V, P = cfg["vocab_size"], cfg["max_position_embeddings"]
    rng = np.random.default_rng(13)
    m = model(name, dtype)
    cache = m.engine.cache
    for lens, decs in (([P - 40, 5, 64, 17], [20, 3, 9, 1]), ([3, 65, 1], [30, 12, 5])):
        seqs = [tiny.prompt(rng, a + d, V) for a, d in zip(lens, decs)]
        refs = [plain_logits(name, s) for s in seqs]
        slots = [m.open_sequence() for _ in seqs]
        got = [[] for _ in seqs]
        out = m.step([(slots[i], seqs[i][:lens[i]]) for i in range(len(seqs))],
                     [list(range(lens[i])) for i in range(len(seqs))]).cpu().numpy()
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
            for i in live:
                if step + 1 == decs[i]:
                    m.close_sequence(slots[i])      # ends earlier: its slot goes back now
        for i in range(len(seqs)):
            g = np.concatenate(got[i])
            for t in range(len(seqs[i])):
                err, bound = tiny.close(g[t], refs[i][t], dtype)
                assert err <= bound, (f"{name} {dtype} batch {lens}: request {i} first wrong at position {t} "
                                      f"(prompt {lens[i]}): {err:.3e} > {bound:.3e}")
        cache.check()
        assert cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_prompts_in_pieces_of_unequal_sizes(name, dtype):
    """Prompts fed in several steps of more than one token each, the sequences of a step with different
    piece sizes and different amounts already cached (pieces that end inside a page, on a page's edge,
    and of one token among long ones): every position's logits as in the whole sequence."""
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(21)
    m = model(name, dtype)
    top = cfg["max_position_embeddings"] - 1
    lens = [min(top, n) for n in (200, 131, 64)]
    seqs = [tiny.prompt(rng, n, cfg["vocab_size"]) for n in lens]
    refs = [plain_logits(name, s) for s in seqs]
    pieces = [[70, 1, 58, 71], [64, 64, 3], [5, 33, 26]]
    slots = [m.open_sequence() for _ in seqs]
    done = [0, 0, 0]
    for step in range(4):
        live = [i for i in range(3) if step < len(pieces[i]) and done[i] < lens[i]]
        if not live:
            break
        runs, want = [], []
        for i in live:
            n = min(pieces[i][step], lens[i] - done[i])
            runs.append((slots[i], seqs[i][done[i]:done[i] + n]))
            want.append(list(range(n)))
        got = m.step(runs, want).cpu().numpy()
        o = 0
        for i, (_, toks) in zip(live, runs):
            check(got[o:o + len(toks)], refs[i][done[i]:done[i] + len(toks)], dtype, f"{name} step {step} sequence {i}")
            o += len(toks)
            done[i] += len(toks)
    for s in slots:
        m.close_sequence(s)
    m.engine.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(dtype):
    """A short prompt, then decoding up to the model's last position."""
    name = "B"
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(14)
    m = model(name, dtype)
    n = cfg["max_position_embeddings"]
    toks = tiny.prompt(rng, n, cfg["vocab_size"])
    ref = plain_logits(name, toks)
    s = m.open_sequence()
    m.step([(s, toks[:4])], [[]])
    for t in range(4, n):
        got = m.step([(s, [toks[t]])]).cpu().numpy()
        err, bound = tiny.close(got[0], ref[t], dtype)
        assert err <= bound, f"{dtype}: first wrong position {t}: {err:.3e} > {bound:.3e}"
    with pytest.raises(Exception):
        m.step([(s, [1])])          # the sequence is full
    m.close_sequence(s)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batch_composition_does_not_change_a_row(dtype):
    name = "A"
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(15)
    m = model(name, dtype)
    a = tiny.prompt(rng, 33, cfg["vocab_size"])
    others = [tiny.prompt(rng, k, cfg["vocab_size"]) for k in (90, 2, 64)]
    s = m.open_sequence()
    alone = m.step([(s, a)], [list(range(33))]).cpu().numpy()
    m.close_sequence(s)
    slots = [m.open_sequence() for _ in range(4)]
    runs = [(slots[0], others[0]), (slots[1], a), (slots[2], others[1]), (slots[3], others[2])]
    out = m.step(runs, [[], list(range(33)), [], []]).cpu().numpy()
    for sl in slots:
        m.close_sequence(sl)
    if dtype == "float32":
        assert np.array_equal(alone, out), "a 32-bit row changed with the batch around it"
    else:
        check(out, alone, dtype, "row in a batch vs alone")


def test_captured_steps_are_kept_up_to_a_limit():
    """Decode steps of the bfloat16 path replay a captured graph per batch size and length bucket; with
    room for two, batches of 1, 2 and 3 in turn keep displacing one another, and every step's logits
    still equal the plain implementation's."""
    name = "B"
    cfg = tiny.TINY[name][0]
    rng = np.random.default_rng(16)
    m = model(name, "bfloat16")
    eng = m.engine
    old, kept = eng.graph_limit, dict(eng._graphs)
    eng.graph_limit = 2
    eng._graphs.clear()
    try:
        seqs = [tiny.prompt(rng, 40, cfg["vocab_size"]) for _ in range(3)]
        refs = [plain_logits(name, t) for t in seqs]
        slots = [m.open_sequence() for _ in seqs]
        m.step([(s, t[:8]) for s, t in zip(slots, seqs)], [[], [], []])
        fed = [8, 8, 8]
        captured = 0
        for rnd in range(18):
            k = (rnd // 3) % 3 + 1                           # sequences 0..k-1 take one token; three steps a size
            out = m.step([(slots[i], [seqs[i][fed[i]]]) for i in range(k)]).cpu().numpy()
            for i in range(k):
                err, bound = tiny.close(out[i], refs[i][fed[i]], "bfloat16")
                assert err <= bound, (rnd, i, err)
                fed[i] += 1
            assert len(eng._graphs) <= 2
            captured += sum(1 for g in eng._graphs.values() if g is not False)
        assert captured > 0, "no step was replayed from a captured graph"
        for s in slots:
            m.close_sequence(s)
    finally:
        eng.graph_limit = old
        eng._graphs.update(kept)
    eng.cache.check()


@pytest.fixture
def fused_layer_for_any_batch():
    """The fused decode layer is taken from 17 or 33 tokens on by default; these tests want it from one."""
    from gopherllm_b200 import ops
    old = ops.DECODE_LAYER_MIN_ROWS, ops.DECODE_LAYER_MIN_CONTEXT, ops.DECODE_LAYER_MIN_ROWS_CUT_TILES
    ops.DECODE_LAYER_MIN_ROWS, ops.DECODE_LAYER_MIN_CONTEXT, ops.DECODE_LAYER_MIN_ROWS_CUT_TILES = 1, 1, 1
    yield ops
    ops.DECODE_LAYER_MIN_ROWS, ops.DECODE_LAYER_MIN_CONTEXT, ops.DECODE_LAYER_MIN_ROWS_CUT_TILES = old


def test_fused_decode_layer_whole_then_one_by_one(fused_layer_for_any_batch):
    """Configuration D through the fused decode layer (forced on for single tokens, steps run kernel by
    kernel and from captured graphs): a prompt, then 60 tokens one by one across a page's edge; and
    the same steps through the separate kernels agree with it within rounding."""
    import gopherllm_b200 as gl
    ops = fused_layer_for_any_batch
    cfg = tiny.TINY["D"][0]
    rng = np.random.default_rng(17)
    toks = tiny.prompt(rng, 200, cfg["vocab_size"])
    ref = plain_logits("D", toks)
    m = gl.load(tiny.folder("D"), dtype="bfloat16", max_tokens=1024)
    launched = []
    real = ops.decode_layer
    ops.decode_layer = lambda *a, **k: (launched.append(a[0].shape[0]), real(*a, **k))[1]
    try:
        s = m.open_sequence()
        got = [m.step([(s, toks[:140])], [list(range(140))]).cpu().numpy()]
        for t in range(140, 200):
            got.append(m.step([(s, [toks[t]])]).cpu().numpy())
        m.close_sequence(s)
    finally:
        ops.decode_layer = real
    assert launched and set(launched) == {1}, "the decode steps did not go through the fused layer"
    got = np.concatenate(got)
    for t in range(200):
        err, bound = tiny.close(got[t], ref[t], "bfloat16")
        assert err <= bound, f"first wrong position {t}: {err:.3e} > {bound:.3e}"
    m.engine.check_device()
    m.close()


def test_fused_decode_layer_unequal_batches(fused_layer_for_any_batch):
    """Unequal prompts in one step, then one token each through the fused layer; shorter requests end
    earlier; a second batch reuses their slots and pages."""
    import gopherllm_b200 as gl
    cfg = tiny.TINY["D"][0]
    V = cfg["vocab_size"]
    rng = np.random.default_rng(18)
    m = gl.load(tiny.folder("D"), dtype="bfloat16", max_tokens=2048)
    cache = m.engine.cache
    for lens, decs in (([250, 5, 64, 17, 130], [40, 3, 9, 1, 66]), ([3, 65, 1], [30, 12, 5])):
        seqs = [tiny.prompt(rng, a + d, V) for a, d in zip(lens, decs)]
        refs = [plain_logits("D", s) for s in seqs]
        slots = [m.open_sequence() for _ in seqs]
        m.step([(slots[i], seqs[i][:lens[i]]) for i in range(len(seqs))], [[] for _ in seqs])
        live = list(range(len(seqs)))
        for step in range(max(decs)):
            live = [i for i in live if step < decs[i]]
            out = m.step([(slots[i], [seqs[i][lens[i] + step]]) for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                err, bound = tiny.close(out[r], refs[i][lens[i] + step], "bfloat16")
                assert err <= bound, f"batch {lens}: request {i} wrong at position {lens[i] + step}: {err:.3e} > {bound:.3e}"
                if step + 1 == decs[i]:
                    m.close_sequence(slots[i])
        cache.check()
        assert cache.slots.held_count == 0 and all(g.pool.held_count == 0 for g in cache.groups)
    m.engine.check_device()
    m.close()


def test_forty_sequences_take_the_fused_decode_layer_by_default():
    """More than 32 tokens a step go through the fused layer without being asked to: 40 sequences of
    unequal lengths, three steps, every row against the plain implementation."""
    import gopherllm_b200 as gl
    from gopherllm_b200 import ops
    cfg = tiny.TINY["D"][0]
    V = cfg["vocab_size"]
    rng = np.random.default_rng(19)
    m = gl.load(tiny.folder("D"), dtype="bfloat16", max_tokens=40 * 128 + 320)
    lens = [int(n) for n in rng.integers(1, 100, size=40)]
    lens[7] = 300                                          # one long sequence: the step's longest decides
    seqs = [tiny.prompt(rng, n + 3, V) for n in lens]
    slots = [m.open_sequence() for _ in seqs]
    launched = []
    real = ops.decode_layer
    ops.decode_layer = lambda *a, **k: (launched.append(a[0].shape[0]), real(*a, **k))[1]
    try:
        for i in range(0, 40, 8):
            m.step([(slots[j], seqs[j][:lens[j]]) for j in range(i, i + 8)], [[] for _ in range(8)])
        outs = [m.step([(slots[i], [seqs[i][lens[i] + step]]) for i in range(40)]).cpu().numpy() for step in range(3)]
    finally:
        ops.decode_layer = real
    assert launched and set(launched) == {40}
    for i in range(0, 40, 3):
        ref = plain_logits("D", seqs[i])
        for step in range(3):
            err, bound = tiny.close(outs[step][i], ref[lens[i] + step], "bfloat16")
            assert err <= bound, (i, step, err, bound)
    for s in slots:
        m.close_sequence(s)
    m.engine.cache.check()
    m.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_later_layers_repeat_the_recorded_launches_of_an_equal_layer(dtype):
    """Six equal layers.  A step records the launches of a layer, compares them with the next layer's
    and repeats them for the rest with those layers' tensors.  The logits must be bit for bit what the
    step gives when every layer walks through its parts, for prompts of unequal lengths in one step and
    for the single-token steps behind them, and they must agree with the plain implementation."""
    import gopherllm_b200 as gl
    from gopherllm_b200 import ops
    cfg = tiny.TINY["E"][0]
    V = cfg["vocab_size"]
    rng = np.random.default_rng(23)
    seqs = [tiny.prompt(rng, n, V) for n in (37, 8, 70)]
    lens = [30, 2, 64]

    def run(repeat):
        ops.REPEAT_LAYERS = repeat
        ops.TAPE_REPEATS = 0
        m = gl.load(tiny.folder("E"), dtype=dtype, max_tokens=3 * 128)
        m.engine.use_graphs = False                        # single-token steps launch their kernels too,
        m.engine.overlap_branches = False                  # on one stream (a fork onto a second one is not repeated)
        slots = [m.open_sequence() for _ in seqs]
        outs = [m.step([(slots[i], seqs[i][:lens[i]]) for i in range(3)], [list(range(n)) for n in lens]).clone()]
        for step in range(5):
            outs.append(m.step([(slots[i], [seqs[i][lens[i] + step]]) for i in range(3)]).clone())
        for s in slots:
            m.close_sequence(s)
        m.engine.check_device()
        m.close()
        return outs, ops.TAPE_REPEATS

    try:
        own, none = run(False)
        rep, count = run(True)
    finally:
        ops.REPEAT_LAYERS = True
    assert none == 0
    assert count >= 6 * 3, f"only {count} repeats in six steps of six layers"
    for a, b in zip(own, rep):
        assert torch.equal(a, b)
    for i in range(3):
        ref = plain_logits("E", seqs[i])
        err, bound = tiny.close(rep[0][sum(lens[:i]):sum(lens[:i + 1])].cpu().numpy(), ref[:lens[i]], dtype)
        assert err <= bound, (i, err, bound)
        for step in range(5):
            err, bound = tiny.close(rep[1 + step][i].cpu().numpy(), ref[lens[i] + step], dtype)
            assert err <= bound, (i, step, err, bound)
