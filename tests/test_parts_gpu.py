"""Each part alone against the plain implementation, and parts defined outside the package."""
import math
import os
import tempfile
from dataclasses import dataclass

import numpy as np
import pytest
import torch

import plain_phi
import tiny

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def harness(requests, dtype, hidden, vocab=50, max_tokens=1024, max_positions=300):
    """A cache and an engine-like context builder for parts run on their own."""
    from gopherllm_b200.cache.sequence_cache import SequenceCache
    from gopherllm_b200.engine.step import Engine

    class Stub:
        class spec:
            pass
    Stub.spec.vocab = vocab
    cache = SequenceCache(requests, max_tokens, max_positions, dtype, DEV)
    eng = Engine(Stub(), cache, dtype, DEV)
    eng.use_graphs = False
    return cache, eng


def context(eng, runs):
    lay, buf, meta = eng.plan(runs, None)
    dev = torch.from_numpy(buf).to(DEV)
    ctx = eng.context(lay, dev, meta)
    for s, n in zip(meta["slots"], meta["new_lens"]):
        eng.cache.commit(s, n)
    return ctx


def rand(shape, seed, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(dtype):
    from gopherllm_b200.config import NormSpec
    from gopherllm_b200.parts import build_norm
    x = rand((9, 160), 1, 2.0).to(DEV)
    for kind, bias in (("layernorm", True), ("rmsnorm", False)):
        n = build_norm(NormSpec(kind, 160, 1e-6, bias=bias))
        params = {k: (1.0 + rand(v.shape, 2, 0.1) if k == "weight" else rand(v.shape, 3, 0.1)).to(DEV)
                  for k, v in n.parameters().items()}
        assert set(params) == ({"weight", "bias"} if bias else {"weight"})
        n.load(params)
        got = n.forward(x, dtype).double().cpu()
        xd = x.double().cpu()
        if kind == "layernorm":
            ref = plain_phi.layer_norm(xd, params["weight"].double().cpu(), params["bias"].double().cpu(), 1e-6)
        else:
            ref = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-6) * params["weight"].double().cpu()
        tol = 1e-5 if dtype == torch.float32 else 2 ** -8
        assert (got - ref).abs().max() <= tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("qk_norm", [False, True])
def test_attention_part_whole_and_in_pieces(dtype, qk_norm):
    """The mixer alone: whole sequence in one step equals prefix + single tokens, and both equal
    the plain formulas (projection, head norm, rotation, scale, causal softmax, projection)."""
    from gopherllm_b200.config import MixerSpec, NormSpec, PositionSpec
    from gopherllm_b200.parts import build_mixer
    D, nH, nKV, hd, rot, T = 96, 6, 2, 32, 16, 70
    spec = MixerSpec("attention", D, nH, nKV, hd, 0, 1 / math.sqrt(hd), True,
                     NormSpec("layernorm", hd, 1e-5, True) if qk_norm else None,
                     PositionSpec("rope", rot, 10000.0))
    mixer = build_mixer(spec)
    P = {k: (rand(v.shape, 10 + i, 0.08) + (1.0 if k.endswith("norm.weight") else 0.0))
         for i, (k, v) in enumerate(sorted(mixer.parameters().items()))}
    store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    P = {k: v.to(store).float() for k, v in P.items()}
    mixer.load({k: (v.to(dtype) if v.dim() == 2 else v).to(DEV) for k, v in P.items()})
    xn = rand((T, D), 5).to(dtype)
    # plain
    xd = xn.double()
    W = {k: v.double() for k, v in P.items()}
    q = (xd @ W["q.weight"].T + W["q.bias"]).reshape(T, nH, hd)
    k = (xd @ W["k.weight"].T + W["k.bias"]).reshape(T, nKV, hd)
    v = (xd @ W["v.weight"].T + W["v.bias"]).reshape(T, nKV, hd)
    if qk_norm:
        q = plain_phi.layer_norm(q, W["q_norm.weight"], W["q_norm.bias"], 1e-5)
        k = plain_phi.layer_norm(k, W["k_norm.weight"], W["k_norm.bias"], 1e-5)
    sin, cos = plain_phi.rope_tables(range(T), rot, 10000.0)
    q, k = plain_phi.apply_rope(q, sin, cos, rot) / math.sqrt(hd), plain_phi.apply_rope(k, sin, cos, rot)
    ref = plain_phi.attention(q, k, v).reshape(T, nH * hd) @ W["out.weight"].T + W["out.bias"]
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for cut in (T, 40):
        cache, eng = harness([mixer.cache_request()], dtype, D)
        s = cache.open()
        outs = []
        pieces = [list(range(cut))] + [[t] for t in range(cut, T)]
        for piece in pieces:
            ctx = context(eng, [(s, [0] * len(piece))])
            add = torch.ones(len(piece), D, device=DEV)
            out = torch.empty(len(piece), D, device=DEV)
            mixer.forward(xn[piece].to(DEV), ctx, cache.view(0), (add,), out)
            outs.append(out.double().cpu() - 1.0)
        got = torch.cat(outs)
        assert (got - ref).abs().max() <= tol * max(1.0, ref.abs().max().item()), cut
        cache.close(s)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("act", ["gelu_new", "gelu", "relu"])
def test_feed_forward_part(dtype, act):
    from gopherllm_b200.config import FeedForwardSpec
    from gopherllm_b200.parts import build_feed_forward
    D, I, T = 72, 200, 11
    ffn = build_feed_forward(FeedForwardSpec("dense", D, I, act, True))
    store = torch.bfloat16 if dtype == torch.bfloat16 else torch.float32
    P = {k: rand(v.shape, 20 + i, 0.1).to(store).float() for i, (k, v) in enumerate(sorted(ffn.parameters().items()))}
    ffn.load({k: (v.to(dtype) if v.dim() == 2 else v).to(DEV) for k, v in P.items()})
    xn = rand((T, D), 6).to(dtype)
    W = {k: v.double() for k, v in P.items()}
    ref = plain_phi.mlp(xn.double(), W["up.weight"], W["up.bias"], W["down.weight"], W["down.bias"], act)
    _, eng = harness([], dtype, D)

    class Ctx:
        act_dtype = dtype
    a0, a1 = rand((T, D), 7).to(DEV), rand((T, D), 8).to(DEV)
    out = torch.empty(T, D, device=DEV)
    ffn.forward(xn.to(DEV), Ctx, (a0, a1), out)
    got = out.double().cpu() - a0.double().cpu() - a1.double().cpu()
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    assert (got - ref).abs().max() <= tol * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_blocks(dtype):
    """The parallel block equals the plain phi block; the sequential arrangement equals its formula."""
    from gopherllm_b200.config import PhiConfig, resolve_architecture
    from gopherllm_b200.config.specs import BlockSpec
    from gopherllm_b200.parts import build_block
    cfg = dict(tiny.TINY_C)
    spec = resolve_architecture("phi").build_spec(PhiConfig.from_dict(cfg))
    bs = spec.layers[0]
    T, D = 50, cfg["hidden_size"]
    pcfg, Wf = plain_phi.read_folder(tiny.folder("C"))
    names = resolve_architecture("phi").tensor_names(PhiConfig.from_dict(cfg))
    x0 = rand((T, D), 9)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for arrangement in ("parallel", "sequential"):
        b = build_block(BlockSpec(arrangement, bs.norm, bs.mixer, bs.ffn, bs.norm if arrangement == "sequential" else None))
        tensors = {}
        for key, ps in b.parameters().items():
            slot, pk = key.split("/")
            src = names.layer(0, "norm" if slot == "norm2" else slot, pk)
            t = Wf[src].float()
            tensors[key] = (t.to(dtype) if ps.kind == "matrix" else t).to(DEV)
        b.load(tensors)
        cache, eng = harness([b.cache_request()], dtype, D)
        s = cache.open()
        x = x0.clone().to(DEV)
        b.forward(x, context(eng, [(s, [0] * T)]), cache.view(0))
        if arrangement == "parallel":
            ref = plain_phi.phi_block(x0.double(), list(range(T)), Wf, 0, pcfg)
        else:
            # x + attn(norm(x)), then + mlp(norm(that)): build it from the plain parts
            zero = {k: torch.zeros_like(v) for k, v in Wf.items() if ".mlp." in k}
            only_attn = plain_phi.phi_block(x0.double(), list(range(T)), {**Wf, **zero}, 0, pcfg)
            pre = "model.layers.0."
            n2 = plain_phi.layer_norm(only_attn, Wf[pre + "input_layernorm.weight"], Wf[pre + "input_layernorm.bias"],
                                      pcfg["layer_norm_eps"])
            ref = only_attn + plain_phi.mlp(n2, Wf[pre + "mlp.fc1.weight"], Wf[pre + "mlp.fc1.bias"],
                                            Wf[pre + "mlp.fc2.weight"], Wf[pre + "mlp.fc2.bias"], pcfg["hidden_act"])
        assert (x.double().cpu() - ref).abs().max() <= tol * max(1.0, ref.abs().max().item()), arrangement


# ---------------------------------------------------------------------------
# parts and an architecture defined here, outside the package
# ---------------------------------------------------------------------------
def define_toy():
    """A mixer with state of its own (an exponential moving sum over a sequence's tokens, one
    state row per sequence), a toy architecture that alternates it with attention, and their
    registration.  Nothing inside gopherllm_b200 is edited."""
    from gopherllm_b200.config import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec,
                                       ScheduleEntry)
    from gopherllm_b200.config.registry import Architecture, register_architecture, resolve_architecture
    from gopherllm_b200.parts import Mixer, ParamSpec, StateRequest, register_mixer

    class EmaMixer(Mixer):
        def __init__(self, spec):
            self.spec, self.decay = spec, float(spec.option("decay", 0.5))

        def parameters(self):
            return {"proj.weight": ParamSpec((self.spec.hidden, self.spec.hidden))}

        def load(self, t):
            self.w = t["proj.weight"]

        def cache_request(self):
            return StateRequest((self.spec.hidden,))

        def forward(self, xn, ctx, cache, add, out):
            starts, lens, slots = ctx.seq_qstart.tolist(), ctx.seq_qlen.tolist(), ctx.seq_slot.tolist()
            y = torch.empty(xn.shape, dtype=torch.float32, device=xn.device)
            for b in range(ctx.n_seqs):
                s = cache.rows[slots[b]]
                for t in range(starts[b], starts[b] + lens[b]):
                    s.mul_(self.decay).add_(xn[t].float())
                    y[t] = s
            res = y @ self.w.float().T
            for a in add:
                res = res + a
            out.copy_(res)
            return out

    if resolve_architecture("toy-ema") is None:
        register_mixer("ema", EmaMixer)

        @dataclass
        class ToyConfig:
            hidden_size: int = 48
            vocab_size: int = 90
            decay: float = 0.5
            torch_dtype: str = "bfloat16"
            initializer_range: float = 0.1

            @classmethod
            def from_dict(cls, d):
                return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

            def to_dict(self):
                return dict(architectures=["ToyEmaForCausalLM"], model_type="toy-ema", **self.__dict__)

        def spec_of(c):
            norm = NormSpec("rmsnorm", c.hidden_size, 1e-5, bias=False)
            ema = MixerSpec("ema", c.hidden_size, extra=(("decay", c.decay),))
            att = MixerSpec("attention", c.hidden_size, 3, 1, 16, 0, 0.25, False, None, PositionSpec("rope", 16, 100.0))
            ffn = FeedForwardSpec("dense", c.hidden_size, 64, "relu", False)
            layers = (BlockSpec("sequential", norm, ema, ffn, norm), BlockSpec("parallel", norm, att, ffn),
                      BlockSpec("sequential", norm, ema, ffn, norm))
            # layer 0 runs twice, each run with state of its own
            sched = (ScheduleEntry(0, 0), ScheduleEntry(1, 1), ScheduleEntry(2, 2), ScheduleEntry(0, 3))
            return ModelSpec(c.hidden_size, c.vocab_size, 128, layers, sched, norm, tie_embeddings=True, head_bias=False)

        class Names:
            embedding, final_norm, head = "emb.weight", "norm_f", "head"

            def __init__(self, c):
                pass

            def layer(self, i, slot, key):
                return f"h.{i}.{slot}.{key}"

        register_architecture(Architecture("toy-ema", ToyConfig, spec_of, Names), aliases=["ToyEma"])
    return resolve_architecture("toy-ema")


def toy_plain(tokens, W, decay):
    """The toy model written out plainly (float64): sequential EMA blocks, one parallel attention block."""
    def rms(x, w):
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w

    def ffn(x, i):
        return torch.relu(x @ W[f"h.{i}.ffn.up.weight"].T) @ W[f"h.{i}.ffn.down.weight"].T

    def ema_block(x, i):
        n = rms(x, W[f"h.{i}.norm.weight"])
        s, ys = torch.zeros(x.shape[1], dtype=x.dtype), []
        for t in range(x.shape[0]):
            s = decay * s + n[t]
            ys.append(s)
        x = x + torch.stack(ys) @ W[f"h.{i}.mixer.proj.weight"].T
        return x + ffn(rms(x, W[f"h.{i}.norm2.weight"]), i)

    def att_block(x, i):
        T = x.shape[0]
        n = rms(x, W[f"h.{i}.norm.weight"])
        q = (n @ W[f"h.{i}.mixer.q.weight"].T).reshape(T, 3, 16)
        k = (n @ W[f"h.{i}.mixer.k.weight"].T).reshape(T, 1, 16)
        v = (n @ W[f"h.{i}.mixer.v.weight"].T).reshape(T, 1, 16)
        sin, cos = plain_phi.rope_tables(range(T), 16, 100.0)
        q, k = plain_phi.apply_rope(q, sin, cos, 16) * 0.25, plain_phi.apply_rope(k, sin, cos, 16)
        a = plain_phi.attention(q, k, v).reshape(T, 48) @ W[f"h.{i}.mixer.out.weight"].T
        return (x + ffn(n, i)) + a

    x = W["emb.weight"][torch.tensor(tokens)]
    for i in (0, 1, 2, 0):
        x = att_block(x, i) if i == 1 else ema_block(x, i)
    return rms(x, W["norm_f.weight"]) @ W["emb.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_mixer_with_state_registered_built_and_stepped(dtype):
    import gopherllm_b200 as gl
    arch = define_toy()
    cfg = arch.config_class()
    folder = tempfile.mkdtemp(prefix="gl_toy_")
    gl.write_random_model(folder, cfg.to_dict(), seed=3)
    m = gl.load(folder, dtype=dtype, max_tokens=512)
    assert m.architecture.name == "toy-ema"
    cache = m.engine.cache
    assert len(cache.groups) == 1 and len(cache._states) == 3          # one attention entry, three state entries
    _, W = plain_phi.read_folder(folder)
    rng = np.random.default_rng(4)
    seqs = [tiny.prompt(rng, n, cfg.vocab_size) for n in (30, 7, 64)]
    refs = [toy_plain(s, W, cfg.decay).numpy() for s in seqs]
    tol = dict(float32=2e-4, bfloat16=3e-2)[dtype]
    for round_ in range(2):                                            # the second round reuses slots: state must restart at zero
        slots = [m.open_sequence() for _ in seqs]
        cut = [20, 3, 64]
        out = m.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
        o = 0
        for i, c in enumerate(cut):
            assert np.abs(out[o:o + c] - refs[i][:c]).max() <= tol * max(1.0, np.abs(refs[i]).max()), (round_, i)
            o += c
        for t in range(max(len(s) - c for s, c in zip(seqs, cut))):
            live = [i for i in range(3) if cut[i] + t < len(seqs[i])]
            out = m.step([(slots[i], [seqs[i][cut[i] + t]]) for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                assert np.abs(out[r] - refs[i][cut[i] + t]).max() <= tol * max(1.0, np.abs(refs[i]).max()), (round_, i, t)
        for sl in slots:
            m.close_sequence(sl)
    got = m.generate(seqs[1], max_tokens=5, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0, stop_tokens=())
    assert len(got.tokens) == 5


# --------------------------------------------------------------------------
# A feed-forward with routing and another position encoding, defined here, registered and run
# without a change to the package: a toy, not anybody's model.
def define_toy_routed():
    from gopherllm_b200.config import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec)
    from gopherllm_b200.config.registry import Architecture, register_architecture, resolve_architecture
    from gopherllm_b200.config.specs import default_schedule
    from gopherllm_b200.parts import FeedForward, ParamSpec, PositionEncoding, register_feed_forward, register_position

    class StretchedRope(PositionEncoding):
        """Rotary angles of position / stretch (tables made with torch, in 64-bit)."""
        def __init__(self, spec):
            self.spec, self.stretch = spec, float(spec.option("stretch", 1.0))

        def tables(self, ctx):
            key = ("stretched", self.spec.rotary_dim, self.spec.theta, self.stretch)
            if key not in ctx.scratch:
                half = self.spec.rotary_dim // 2
                inv = self.spec.theta ** (-torch.arange(half, dtype=torch.float64, device=ctx.device) * 2 / self.spec.rotary_dim)
                ang = (ctx.tok_pos.double() / self.stretch)[:, None] * inv[None, :]
                ctx.scratch[key] = (ang.cos().float().contiguous(), ang.sin().float().contiguous())
            return ctx.scratch[key]

    class TopOneExperts(FeedForward):
        """Router logits and their softmax in 32-bit; a token goes to its best expert and the result is
        weighted with that expert's probability."""
        def __init__(self, spec):
            self.spec, self.n = spec, int(spec.option("experts", 2))

        def parameters(self):
            s = self.spec
            return {"router.weight": ParamSpec((self.n, s.hidden)),
                    "up.weight": ParamSpec((self.n * s.intermediate, s.hidden)),
                    "down.weight": ParamSpec((self.n * s.hidden, s.intermediate))}

        def load(self, t):
            s = self.spec
            self.router = t["router.weight"]
            self.up = t["up.weight"].reshape(self.n, s.intermediate, s.hidden)
            self.down = t["down.weight"].reshape(self.n, s.hidden, s.intermediate)

        def forward(self, xn, ctx, add, out):
            p = torch.softmax(xn.float() @ self.router.float().T, -1)
            gate, choice = p.max(-1)
            res = torch.zeros(xn.shape, dtype=torch.float32, device=xn.device)
            for e in range(self.n):
                rows = (choice == e).nonzero().flatten()
                if rows.numel():
                    h = torch.relu(xn[rows].float() @ self.up[e].float().T).to(xn.dtype).float()
                    res[rows] = gate[rows, None] * (h @ self.down[e].float().T)
            for a in add:
                res = res + a
            out.copy_(res)
            return out

    if resolve_architecture("toy-routed") is None:
        register_position("stretched_rope", StretchedRope)
        register_feed_forward("top_one_experts", TopOneExperts)

        @dataclass
        class RoutedConfig:
            hidden_size: int = 40
            vocab_size: int = 77
            experts: int = 3
            stretch: float = 4.0
            torch_dtype: str = "bfloat16"
            initializer_range: float = 0.2

            @classmethod
            def from_dict(cls, d):
                return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

            def to_dict(self):
                return dict(architectures=["ToyRoutedForCausalLM"], model_type="toy-routed", **self.__dict__)

        def spec_of(c):
            norm = NormSpec("layernorm", c.hidden_size, 1e-6, bias=True)
            pos = PositionSpec("stretched_rope", 8, 50.0, extra=(("stretch", c.stretch),))
            att = MixerSpec("attention", c.hidden_size, 2, 2, 16, 0, 0.25, True, None, pos)
            ffn = FeedForwardSpec("top_one_experts", c.hidden_size, 24, "relu", False, extra=(("experts", c.experts),))
            layers = (BlockSpec("parallel", norm, att, ffn), BlockSpec("sequential", norm, att, ffn, norm))
            return ModelSpec(c.hidden_size, c.vocab_size, 256, layers, default_schedule(2), norm,
                             tie_embeddings=False, head_bias=True)

        class Names:
            embedding, final_norm, head = "emb.weight", "norm_f", "head"

            def __init__(self, c):
                pass

            def layer(self, i, slot, key):
                return f"h.{i}.{slot}.{key}"

        register_architecture(Architecture("toy-routed", RoutedConfig, spec_of, Names), aliases=["ToyRouted"])
    return resolve_architecture("toy-routed")


def toy_routed_plain(tokens, W, cfg, act_dtype):
    """The routed toy written out plainly in 64-bit (the hidden activations rounded where the part
    rounds them, so that a token's choice of expert is the only thing rounding can flip)."""
    def ln(x, pre):
        return plain_phi.layer_norm(x, W[pre + ".weight"], W[pre + ".bias"], 1e-6)

    def ffn(n, i):
        nn = n.to(act_dtype).double()
        p = torch.softmax(nn.float() @ W[f"h.{i}.ffn.router.weight"].float().T, -1).double()
        gate, choice = p.max(-1)
        up = W[f"h.{i}.ffn.up.weight"].reshape(cfg.experts, 24, cfg.hidden_size)
        down = W[f"h.{i}.ffn.down.weight"].reshape(cfg.experts, cfg.hidden_size, 24)
        out = torch.zeros_like(n)
        for t in range(n.shape[0]):
            e = int(choice[t])
            h = torch.relu(nn[t] @ up[e].T).to(act_dtype).double()
            out[t] = gate[t] * (h @ down[e].T)
        return out

    def att(n, i):
        T = n.shape[0]
        qkv = lambda k: n @ W[f"h.{i}.mixer.{k}.weight"].T + W[f"h.{i}.mixer.{k}.bias"]
        q, k, v = (qkv(s).reshape(T, 2, 16) for s in "qkv")
        half = 4
        inv = 50.0 ** (-torch.arange(half, dtype=torch.float64) * 2 / 8)
        ang = (torch.arange(T, dtype=torch.float64) / cfg.stretch)[:, None] * inv[None, :]
        sin, cos = ang.sin(), ang.cos()
        q, k = plain_phi.apply_rope(q, sin, cos, 8) * 0.25, plain_phi.apply_rope(k, sin, cos, 8)
        return plain_phi.attention(q, k, v).reshape(T, 32) @ W[f"h.{i}.mixer.out.weight"].T + W[f"h.{i}.mixer.out.bias"]

    x = W["emb.weight"][torch.tensor(tokens)]
    n = ln(x, "h.0.norm")
    x = (x + ffn(n, 0)) + att(n, 0)
    x = x + att(ln(x, "h.1.norm"), 1)
    x = x + ffn(ln(x, "h.1.norm2"), 1)
    return ln(x, "norm_f") @ W["head.weight"].T + W["head.bias"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_routed_feed_forward_and_position_registered_built_and_stepped(dtype):
    import gopherllm_b200 as gl
    arch = define_toy_routed()
    cfg = arch.config_class()
    folder = tempfile.mkdtemp(prefix="gl_toy_routed_")
    gl.write_random_model(folder, cfg.to_dict(), seed=5)
    m = gl.load(folder, dtype=dtype, max_tokens=512)
    assert m.architecture.name == "toy-routed"
    _, W = plain_phi.read_folder(folder)
    rng = np.random.default_rng(6)
    seqs = [tiny.prompt(rng, n, cfg.vocab_size) for n in (40, 9)]
    act = torch.float32 if dtype == "float32" else torch.bfloat16
    refs = [toy_routed_plain(s, W, cfg, act).numpy() for s in seqs]
    tol = dict(float32=2e-4, bfloat16=3e-2)[dtype]
    slots = [m.open_sequence() for _ in seqs]
    cut = [25, 4]
    out = m.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
    # a token whose two best experts are nearly tied may go either way under rounding: compare the others
    def close(got, ref):
        return np.abs(got - ref).max() <= tol * max(1.0, np.abs(ref).max())
    rows, o, bad = 0, 0, 0
    for i, c in enumerate(cut):
        for t in range(c):
            rows += 1
            bad += not close(out[o + t], refs[i][t])
        o += c
    for t in range(max(len(s) - c for s, c in zip(seqs, cut))):
        live = [i for i in range(2) if cut[i] + t < len(seqs[i])]
        got = m.step([(slots[i], [seqs[i][cut[i] + t]]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            rows += 1
            bad += not close(got[r], refs[i][cut[i] + t])
    for sl in slots:
        m.close_sequence(sl)
    assert bad == 0 if dtype == "float32" else bad <= rows // 10, (bad, rows)


# --------------------------------------------------------------------------
# A block arrangement of its own (a norm after the mixer as well as before it), learned absolute
# positions and scaled, soft-capped logits: a toy again, registered and run without a change to
# the package.
def define_toy_sandwich():
    from gopherllm_b200.config import (BlockSpec, FeedForwardSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec)
    from gopherllm_b200.config.registry import Architecture, register_architecture, resolve_architecture
    from gopherllm_b200.config.specs import default_schedule
    from gopherllm_b200.parts import AssembledBlock, build_norm, register_block

    class SandwichBlock(AssembledBlock):
        """x <- x + post_norm(mixer(norm(x))); x <- x + ffn(norm2(x)).  One child more than the usual
        four; parameters, loading and the capture flag come from ``children``."""

        def __init__(self, spec):
            super().__init__(spec)
            self.post_norm = build_norm(spec.option("post_norm"))

        def children(self):
            c = super().children()
            c["post_norm"] = self.post_norm
            return c

        def forward(self, x, ctx, cache):
            h = torch.empty_like(x)
            self.mixer.forward(self.norm.forward(x, ctx.act_dtype), ctx, cache, (), h)
            x.add_(self.post_norm.forward(h, torch.float32))
            self.ffn.forward(self.norm2.forward(x, ctx.act_dtype), ctx, (x,), x)
            return x

    if resolve_architecture("toy-sandwich") is None:
        register_block("sandwich", SandwichBlock)

        @dataclass
        class SandwichConfig:
            hidden_size: int = 56
            vocab_size: int = 83
            positions: int = 96
            torch_dtype: str = "bfloat16"
            initializer_range: float = 0.15

            @classmethod
            def from_dict(cls, d):
                return cls(**{k: v for k, v in d.items() if k in cls.__dataclass_fields__})

            def to_dict(self):
                return dict(architectures=["ToySandwichForCausalLM"], model_type="toy-sandwich", **self.__dict__)

        def spec_of(c):
            norm = NormSpec("layernorm", c.hidden_size, 1e-5, bias=True)
            post = NormSpec("rmsnorm", c.hidden_size, 1e-6, bias=False)
            att = MixerSpec("attention", c.hidden_size, 2, 1, 32, 0, 32 ** -0.5, False, None, PositionSpec("none"))
            ffn = FeedForwardSpec("dense", c.hidden_size, 72, "gelu", True)
            block = BlockSpec("sandwich", norm, att, ffn, norm, extra=(("post_norm", post),))
            return ModelSpec(c.hidden_size, c.vocab_size, c.positions, (block, block), default_schedule(2), norm,
                             tie_embeddings=False, head_bias=False, embedding_scale=2.0,
                             position_table=c.positions, logit_scale=0.5, logit_softcap=3.0)

        class Names:
            embedding, final_norm, head, positions = "wte.weight", "ln_f", "head", "wpe.weight"

            def __init__(self, c):
                pass

            def layer(self, i, slot, key):
                return f"h.{i}.{slot}.{key}"

        register_architecture(Architecture("toy-sandwich", SandwichConfig, spec_of, Names), aliases=["ToySandwich"])
    return resolve_architecture("toy-sandwich")


def toy_sandwich_plain(tokens, W):
    T = len(tokens)
    x = 2.0 * W["wte.weight"][torch.tensor(tokens)] + W["wpe.weight"][:T]
    for i in range(2):
        p = f"h.{i}."
        n = plain_phi.layer_norm(x, W[p + "norm.weight"], W[p + "norm.bias"], 1e-5)
        q = (n @ W[p + "mixer.q.weight"].T).reshape(T, 2, 32) * 32 ** -0.5
        k = (n @ W[p + "mixer.k.weight"].T).reshape(T, 1, 32)
        v = (n @ W[p + "mixer.v.weight"].T).reshape(T, 1, 32)
        h = plain_phi.attention(q, k, v).reshape(T, 64) @ W[p + "mixer.out.weight"].T
        x = x + h / torch.sqrt((h * h).mean(-1, keepdim=True) + 1e-6) * W[p + "post_norm.weight"]
        n2 = plain_phi.layer_norm(x, W[p + "norm2.weight"], W[p + "norm2.bias"], 1e-5)
        x = x + plain_phi.mlp(n2, W[p + "ffn.up.weight"], W[p + "ffn.up.bias"], W[p + "ffn.down.weight"],
                              W[p + "ffn.down.bias"], "gelu")
    logits = plain_phi.layer_norm(x, W["ln_f.weight"], W["ln_f.bias"], 1e-5) @ W["head.weight"].T
    return 3.0 * torch.tanh(logits * 0.5 / 3.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_block_with_a_norm_after_its_mixer_positions_table_and_capped_logits(dtype):
    import gopherllm_b200 as gl
    arch = define_toy_sandwich()
    cfg = arch.config_class()
    folder = tempfile.mkdtemp(prefix="gl_toy_sandwich_")
    gl.write_random_model(folder, cfg.to_dict(), seed=8)
    m = gl.load(folder, dtype=dtype, max_tokens=512)
    assert m.architecture.name == "toy-sandwich"
    keys = m.engine.model.parameters()
    assert "layers/1/post_norm/weight" in keys and "positions" in keys
    _, W = plain_phi.read_folder(folder)
    assert "h.1.post_norm.weight" in W and "wpe.weight" in W
    rng = np.random.default_rng(9)
    seqs = [tiny.prompt(rng, n, cfg.vocab_size) for n in (70, 11)]
    refs = [toy_sandwich_plain(s, W).numpy() for s in seqs]
    assert max(np.abs(r).max() for r in refs) > 1.0             # the cap is at work
    tol = dict(float32=2e-4, bfloat16=3e-2)[dtype]
    slots = [m.open_sequence() for _ in seqs]
    cut = [50, 6]
    out = m.step([(sl, s[:c]) for sl, s, c in zip(slots, seqs, cut)], [list(range(c)) for c in cut]).cpu().numpy()
    o = 0
    for i, c in enumerate(cut):
        assert np.abs(out[o:o + c] - refs[i][:c]).max() <= tol * max(1.0, np.abs(refs[i]).max()), i
        o += c
    for t in range(max(len(s) - c for s, c in zip(seqs, cut))):          # decode steps (captured in bfloat16)
        live = [i for i in range(2) if cut[i] + t < len(seqs[i])]
        got = m.step([(slots[i], [seqs[i][cut[i] + t]]) for i in live]).cpu().numpy()
        for r, i in enumerate(live):
            assert np.abs(got[r] - refs[i][cut[i] + t]).max() <= tol * max(1.0, np.abs(refs[i]).max()), (i, t)
    for sl in slots:
        m.close_sequence(sl)
    m.engine.cache.check()
