"""Each kernel alone against a plain reference, at sizes other than the models'."""
import math

import numpy as np
import pytest
import torch

import plain_phi

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


def ops():
    from gopherllm_b200 import ops as o
    return o


def gelu_ref(x, act):
    if act in (None, "none"):
        return x
    return plain_phi.ACTIVATIONS[act](x)


def ref_linear(a, w, bias, act, add0, add1):
    v = a.double() @ w.double().T
    if bias is not None:
        v = v + bias.double()
    v = gelu_ref(v, act)
    for t in (add0, add1):
        if t is not None:
            v = v + t.double()
    return v


def rnd(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


# --------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 7, 5), (5, 77, 33), (130, 200, 96), (64, 64, 16), (3, 1000, 416)])
@pytest.mark.parametrize("adt,wdt", [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                     (torch.bfloat16, torch.float32), (torch.float32, torch.bfloat16)])
def test_gemm_simt(M, N, K, adt, wdt):
    o = ops()
    a, w = rnd(M, K, dtype=adt), rnd(N, K, dtype=wdt, seed=1)
    bias, add0, add1 = rnd(N, seed=2), rnd(M, N, seed=3), rnd(M, N, seed=4)
    for act in (None, "gelu_new", "gelu", "relu"):
        got = o.gemm_simt(a, w, bias, act, add0, add1, out_dtype=torch.float32)
        ref = ref_linear(a, w, bias, act, add0, add1)
        assert (got.double() - ref).abs().max() <= 2e-5 * max(1.0, ref.abs().max().item())
    got = o.gemm_simt(a, w, out_dtype=torch.bfloat16)
    ref = ref_linear(a, w, None, None, None, None)
    assert (got.double() - ref).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max().item())
    # in place on the residual stream
    x = add0.clone()
    o.gemm_simt(a, w, bias, None, x, add1, out=x)
    assert (x.double() - ref_linear(a, w, bias, None, add0, add1)).abs().max() <= 2e-5 * max(1.0, ref.abs().max().item())


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("N,K", [(40, 160), (1000, 200), (2560, 2560), (130, 4104)])
def test_gemm_skinny(M, N, K):
    o = ops()
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    bias, add0, add1 = rnd(N, seed=2), rnd(M, N, seed=3), rnd(M, N, seed=4)
    for split in (0, 1, 2, 4, 8):
        for act in (None, "gelu_new"):
            got = o.gemm_skinny(a, w, bias, act, add0, add1, out_dtype=torch.float32, split_k=split)
            ref = ref_linear(a, w, bias, act, add0, add1)
            err = (got.double() - ref).abs().max().item()
            assert err <= 3e-5 * max(1.0, ref.abs().max().item()), (split, act, err)
    got = o.gemm_skinny(a, w, bias, "gelu", out_dtype=torch.bfloat16)
    ref = ref_linear(a, w, bias, "gelu", None, None)
    assert (got.double() - ref).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max().item())
    with pytest.raises(Exception):
        o.gemm_skinny(rnd(65, K, dtype=torch.bfloat16), w)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 128, 128), (65, 40, 160), (200, 1000, 200),
                                   (300, 777 * 8, 416), (2048, 2560, 2560), (1000, 7680, 2568),
                                   (6405, 200, 2560)])      # (rows enough for several groups of row tiles, the last one partial)
def test_gemm_tcgen05(M, N, K):
    o = ops()
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    bias, add0, add1 = rnd(N, seed=2), rnd(M, N, seed=3), rnd(M, N, seed=4)
    ref = ref_linear(a, w, bias, "gelu_new", add0, add1)
    for tile in (0, 64, 128, 160, 192, 256, 1160, 1192, 1256):
        got = o.gemm_tcgen05(a, w, bias, "gelu_new", add0, add1, out_dtype=torch.float32, tile_n=tile)
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_tcgen05"] == 0, "a bounded wait ran out"
        err = (got.double() - ref).abs().max().item()
        assert err <= 3e-5 * max(1.0, ref.abs().max().item()), (tile, err)
    for act in (None, "gelu_new"):
        for tile in (0, 64, 192, 1192, 1256):
            got = o.gemm_tcgen05(a, w, bias, act, out_dtype=torch.bfloat16, tile_n=tile)
            ref = ref_linear(a, w, bias, act, None, None)
            assert (got.double() - ref).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max().item()), (act, tile)
    for tile in (0, 160, 256, 1160, 1256):
        got = o.gemm_tcgen05(a, w, bias, "gelu", out_dtype=torch.float32, tile_n=tile)    # the plain TMA store
        ref = ref_linear(a, w, bias, "gelu", None, None)
        assert (got.double() - ref).abs().max() <= 3e-5 * max(1.0, ref.abs().max().item()), tile
    ref = ref_linear(a, w, bias, None, None, None)
    x = add0.clone()                                                   # in place on the residual stream
    o.gemm_tcgen05(a, w, bias, None, x, add1, out=x)
    assert (x.double() - ref_linear(a, w, bias, None, add0, add1)).abs().max() <= 3e-5 * max(1.0, ref.abs().max().item())
    want = ref_linear(a, w, bias, "relu", add0, None)
    for tile in (0, 1160, 1256):
        x = add0.clone()                                               # out = out + product: the add-reduction path
        o.gemm_tcgen05(a, w, bias, "relu", x, out=x, tile_n=tile)
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_tcgen05"] == 0
        assert (x.double() - want).abs().max() <= 3e-5 * max(1.0, want.abs().max().item()), tile


@pytest.mark.parametrize("M,N,K", [(1024, 2560, 1024), (520, 1300, 4104), (2048, 2560, 2560)])
def test_gemm_tcgen05_cut_tiles(M, N, K):
    """out = out + product at sizes whose tiles fill the SMs unevenly: the blocks share (tile, k-block)
    units equally and tiles cut between blocks are summed by the add-reduction; the bias counts once."""
    o = ops()
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    bias, x0 = rnd(N, seed=2), rnd(M, N, seed=3)
    want = ref_linear(a, w, bias, None, x0, None)
    o.gemm_tcgen05_cut_tiles(1)
    try:
        _cut_tiles_checks(o, a, w, bias, x0, want, M, N, K)
    finally:
        o.gemm_tcgen05_cut_tiles(0)


def _cut_tiles_checks(o, a, w, bias, x0, want, M, N, K):
    for tile in (0, 128, 256, 1160):
        x = x0.clone()
        o.gemm_tcgen05(a, w, bias, None, x, out=x, tile_n=tile)
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_tcgen05"] == 0, "a bounded wait ran out"
        err = (x.double() - want).abs().max().item()
        assert err <= 3e-5 * max(1.0, want.abs().max().item()), (tile, err)
    # one weight far along K reaches one column exactly, whichever block holds its k-block
    a1 = torch.ones(M, K, dtype=torch.bfloat16, device=DEV)
    for (n, k) in [(0, 0), (N - 1, K - 1), (N // 2 + 3, K // 2 + 9), (255, 64), (256, 63)]:
        w1 = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
        w1[n, k] = 3.0
        x = torch.zeros(M, N, device=DEV)
        o.gemm_tcgen05(a1, w1, None, None, x, out=x)
        expect = torch.zeros(M, N, device=DEV)
        expect[:, n] = 3.0
        assert torch.equal(x, expect), (n, k)


@pytest.mark.parametrize("M,N,K1,K2", [(300, 200, 96, 160), (130, 520, 200, 1096), (2048, 2560, 2560, 10240)])
def test_gemm_tcgen05_two_products_one_tile(M, N, K1, K2):
    """out = out + a1 w1^T + b1 + a2 w2^T + b2: two branches' last products as one product over the
    joined K (K1 need not fill its last k-block), against the two run one after the other in 64-bit."""
    o = ops()
    a1, w1 = rnd(M, K1, dtype=torch.bfloat16), rnd(N, K1, dtype=torch.bfloat16, scale=0.05, seed=1)
    a2, w2 = rnd(M, K2, dtype=torch.bfloat16, seed=5), rnd(N, K2, dtype=torch.bfloat16, scale=0.05, seed=6)
    b1, b2, x0 = rnd(N, seed=2), rnd(N, seed=7), rnd(M, N, seed=3)
    want = ref_linear(a1, w1, b1, None, x0, None) + ref_linear(a2, w2, b2, None, None, None)
    for tile in (0, 128, 256, 1160):
        x = x0.clone()
        o.gemm_tcgen05(a1, w1, b1, None, x, out=x, tile_n=tile, second=(a2, w2, b2))
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_tcgen05"] == 0, "a bounded wait ran out"
        err = (x.double() - want).abs().max().item()
        assert err <= 3e-5 * max(1.0, want.abs().max().item()), (tile, err)
    x = x0.clone()
    o.linear_pair(a1, w1, b1, a2, w2, None, add0=x, out=x)                 # the dispatching call, one bias missing
    want = ref_linear(a1, w1, b1, None, x0, None) + ref_linear(a2, w2, None, None, None, None)
    assert (x.double() - want).abs().max() <= 3e-5 * max(1.0, want.abs().max().item())
    x = x0[:8].clone()                                                      # few rows: one after the other
    o.linear_pair(a1[:8], w1, b1, a2[:8], w2, b2, add0=x, out=x)
    want = ref_linear(a1[:8], w1, b1, None, x0[:8], None) + ref_linear(a2[:8], w2, b2, None, None, None)
    assert (x.double() - want).abs().max() <= 3e-5 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("M,N,NB,K", [(300, 200, 520, 96), (130, 528, 72, 1096), (2048, 7680, 10240, 2560),
                                      (5700, 136, 328, 2560)])
def test_gemm_tcgen05_two_sets_of_columns(M, N, NB, K):
    """(a w^T + b, act(a wB^T + bB)) from one launch: the tiles of the second set follow the first's,
    each with its own bias, activation, width and output; against each product alone in 64-bit, and
    bit for bit against the same kernel run once per set."""
    o = ops()
    a = rnd(M, K, dtype=torch.bfloat16)
    w, wb = rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1), rnd(NB, K, dtype=torch.bfloat16, scale=0.05, seed=4)
    b, bb = rnd(N, seed=2), rnd(NB, seed=5)
    want, want_b = ref_linear(a, w, b, None, None, None), ref_linear(a, wb, bb, "gelu_new", None, None)
    for tile in (0, 64, 128, 192, 256, 1256):
        y, yb = o.gemm_tcgen05(a, w, b, None, tile_n=tile, fork=(wb, bb, "gelu_new"))
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_tcgen05"] == 0, "a bounded wait ran out"
        assert y.shape == (M, N) and yb.shape == (M, NB) and y.dtype == yb.dtype == torch.bfloat16
        for got, ref in ((y, want), (yb, want_b)):
            err = (got.double() - ref).abs().max().item()
            assert err <= 2 ** -8 * max(1.0, ref.abs().max().item()), (tile, err)
        assert torch.equal(y, o.gemm_tcgen05(a, w, b, None, tile_n=tile))
        assert torch.equal(yb, o.gemm_tcgen05(a, wb, bb, "gelu_new", tile_n=tile))
    y, yb = o.linear_fork(a, w, None, None, wb, bb, "gelu_new", torch.float32)       # 32-bit outputs, one bias missing
    assert (y.double() - ref_linear(a, w, None, None, None, None)).abs().max() <= 3e-5 * max(1.0, want.abs().max().item())
    assert (yb.double() - want_b).abs().max() <= 3e-5 * max(1.0, want_b.abs().max().item())
    y, yb = o.linear_fork(a[:8], w, b, None, wb, bb, "gelu_new")                      # few rows: one after the other
    assert (y.double() - want[:8]).abs().max() <= 2 ** -8 * max(1.0, want.abs().max().item())
    assert (yb.double() - want_b[:8]).abs().max() <= 2 ** -8 * max(1.0, want_b.abs().max().item())


def test_gemm_tcgen05_one_weight_stands_out():
    """A single large weight must reach exactly one output column, wherever it sits in K and N."""
    o = ops()
    M, N, K = 130, 520, 1096
    a = torch.ones(M, K, dtype=torch.bfloat16, device=DEV)
    for (n, k) in [(0, 0), (519, 1095), (77, 1029), (256, 63), (255, 64), (128, 15), (127, 16), (511, 1088)]:
        w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
        w[n, k] = 3.0
        for tile in (64, 128, 160, 192, 256, 1160, 1192, 1256):
            got = o.gemm_tcgen05(a, w, out_dtype=torch.float32, tile_n=tile)
            want = torch.zeros(M, N, device=DEV)
            want[:, n] = 3.0
            assert torch.equal(got, want), (n, k, tile)
    # and a single activation reaches exactly one row
    w = torch.ones(N, K, dtype=torch.bfloat16, device=DEV)
    for (m, k) in [(0, 0), (129, 1095), (64, 520), (127, 7), (128, 8)]:
        a = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
        a[m, k] = 2.0
        for tile in (0, 1192):
            got = o.gemm_tcgen05(a, w, out_dtype=torch.float32, tile_n=tile)
            want = torch.zeros(M, N, device=DEV)
            want[m, :] = 2.0
            assert torch.equal(got, want), (m, k, tile)


@pytest.mark.parametrize("M,N,K1,K2", [(8, 200, 64, 160), (1, 2560, 2560, 10240), (64, 520, 192, 1096), (17, 77, 128, 8)])
def test_gemm_skinny_two_products_one_output(M, N, K1, K2):
    o = ops()
    a1, w1 = rnd(M, K1, dtype=torch.bfloat16), rnd(N, K1, dtype=torch.bfloat16, scale=0.05, seed=1)
    a2, w2 = rnd(M, K2, dtype=torch.bfloat16, seed=5), rnd(N, K2, dtype=torch.bfloat16, scale=0.05, seed=6)
    b1, b2, x0 = rnd(N, seed=2), rnd(N, seed=7), rnd(M, N, seed=3)
    want = ref_linear(a1, w1, b1, None, x0, None) + ref_linear(a2, w2, b2, None, None, None)
    for split in (0, 1, 2, 4, 8):
        x = x0.clone()
        o.gemm_skinny(a1, w1, b1, None, x, out=x, split_k=split, second=(a2, w2, b2))
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_skinny"] == 0, "a bounded wait ran out"
        err = (x.double() - want).abs().max().item()
        assert err <= 3e-5 * max(1.0, want.abs().max().item()), (split, err)
    x = x0.clone()
    o.linear_pair(a2, w2, b2, a1, w1, b1, add0=x, out=x)           # K2 first: the dispatcher puts whole stages first
    assert (x.double() - want).abs().max() <= 3e-5 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("M,N,K", [(17, 128, 64), (64, 200, 416), (33, 777, 2568), (40, 2560, 2560), (64, 7680, 2560),
                                   (20, 1000, 200), (64, 64, 8), (31, 2560, 12800)])
def test_gemm_stream(M, N, K):
    """The tensor-core weight-streaming product (weights as the 128-row operand) for 17 to 64 rows:
    every split of K over a cluster, both output types, awkward N and K."""
    o = ops()
    a, w = rnd(M, K, dtype=torch.bfloat16), rnd(N, K, dtype=torch.bfloat16, scale=0.05, seed=1)
    bias, add0, add1 = rnd(N, seed=2), rnd(M, N, seed=3), rnd(M, N, seed=4)
    ref = ref_linear(a, w, bias, "gelu_new", add0, add1)
    chunks = -(-K // 64)
    for split in (0, 1, 2, 3, 5, 8, 16):
        if split > chunks:
            continue
        got = o.gemm_stream(a, w, bias, "gelu_new", add0, add1, out_dtype=torch.float32, split_k=split)
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_stream"] == 0, "a bounded wait ran out"
        err = (got.double() - ref).abs().max().item()
        assert err <= 2e-3 * max(1.0, ref.abs().max().item()), (split, err)
    got = o.gemm_stream(a, w, None, None, out_dtype=torch.bfloat16)
    ref = ref_linear(a, w, None, None, None, None)
    assert (got.double() - ref).abs().max().item() <= 2 ** -7 * max(1.0, ref.abs().max().item())
    # the same bits from run to run: the parts are added in rank order
    again = o.gemm_stream(a, w, None, None, out_dtype=torch.bfloat16)
    assert torch.equal(got, again)


@pytest.mark.parametrize("M,N,K1,K2", [(17, 128, 64, 64), (64, 2560, 2560, 10240), (40, 200, 128, 200), (33, 777, 320, 8)])
def test_gemm_stream_two_products_one_output(M, N, K1, K2):
    o = ops()
    a, w = rnd(M, K1, dtype=torch.bfloat16), rnd(N, K1, dtype=torch.bfloat16, scale=0.05, seed=1)
    a2, w2 = rnd(M, K2, dtype=torch.bfloat16, seed=5), rnd(N, K2, dtype=torch.bfloat16, scale=0.05, seed=6)
    bias, bias2, add0 = rnd(N, seed=2), rnd(N, seed=7), rnd(M, N, seed=3)
    ref = a.double() @ w.double().T + a2.double() @ w2.double().T + bias.double() + bias2.double() + add0.double()
    for split in (0, 1, 4, 7):
        out = add0.clone()
        o.gemm_stream(a, w, bias, None, out, None, torch.float32, out, split_k=split, second=(a2, w2, bias2))
        torch.cuda.synchronize()
        assert o.wait_failures()["libgl_gemm_stream"] == 0, "a bounded wait ran out"
        assert (out.double() - ref).abs().max().item() <= 2e-3 * max(1.0, ref.abs().max().item()), split


def test_gemm_stream_one_weight_stands_out():
    """One large weight at a far corner (last row tile, last k-block of the second product): every token's
    output in that column must carry it; a lost tile, stage or part would not."""
    o = ops()
    M, N, K1, K2 = 48, 2560 + 40, 2560, 1000
    a, a2 = rnd(M, K1, dtype=torch.bfloat16), rnd(M, K2, dtype=torch.bfloat16, seed=5)
    w = torch.zeros(N, K1, dtype=torch.bfloat16, device=DEV)
    w2 = torch.zeros(N, K2, dtype=torch.bfloat16, device=DEV)
    w2[N - 1, K2 - 1] = 64.0
    w[5, 0] = -32.0
    out = torch.zeros(M, N, device=DEV)
    o.gemm_stream(a, w, None, None, None, None, torch.float32, out, second=(a2, w2, None))
    torch.cuda.synchronize()
    want = torch.zeros(M, N, dtype=torch.float64)
    want[:, N - 1] = 64.0 * a2[:, K2 - 1].double().cpu()
    want[:, 5] = -32.0 * a[:, 0].double().cpu()
    assert torch.equal(out.double().cpu(), want)


def test_gemm_skinny_one_weight_stands_out():
    """A single large weight far along K must reach exactly one output."""
    o = ops()
    M, N, K = 8, 192, 2048
    a = torch.ones(M, K, dtype=torch.bfloat16, device=DEV)
    for (n, k) in [(0, 0), (191, 2047), (77, 1029), (64, 31), (63, 32)]:
        w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
        w[n, k] = 3.0
        for split in (1, 2, 4, 8):
            got = o.gemm_skinny(a, w, out_dtype=torch.float32, split_k=split)
            want = torch.zeros(M, N, device=DEV)
            want[:, n] = 3.0
            assert torch.equal(got, want), (n, k, split)


# --------------------------------------------------------------------------
@pytest.mark.parametrize("D", [5, 64, 160, 2560, 3000])
def test_norm_and_embed(D):
    o = ops()
    x = rnd(11, D, scale=3.0) + 0.7
    g, b = rnd(D, seed=1) + 1.0, rnd(D, seed=2)
    for eps in (1e-5, 1e-6):
        ref = plain_phi.layer_norm(x.double().cpu(), g.double().cpu(), b.double().cpu(), eps)
        got = o.norm(x, g, b, eps, torch.float32)
        assert (got.double().cpu() - ref).abs().max() <= 1e-5 * max(1.0, ref.abs().max().item())
        rows = torch.tensor([10, 0, 3, 3], dtype=torch.int32, device=DEV)
        got = o.norm(x, g, b, eps, torch.bfloat16, rows=rows)
        assert (got.double().cpu() - ref[[10, 0, 3, 3]]).abs().max() <= 2 ** -8 * max(1.0, ref.abs().max().item())
        xr = x.double().cpu()
        rms = xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + eps) * g.double().cpu()
        got = o.norm(x, g, None, eps, torch.float32, rms=True)
        assert (got.double().cpu() - rms).abs().max() <= 1e-5 * max(1.0, rms.abs().max().item())
    for dt in (torch.float32, torch.bfloat16):
        table = rnd(37, D, dtype=dt, seed=5)
        toks = torch.tensor([36, 0, 5, 5, 17], dtype=torch.int32, device=DEV)
        assert torch.equal(o.embed(table, toks), table[toks.long()].float())
        assert torch.equal(o.embed(table, toks, scale=2.0), table[toks.long()].float() * 2.0)


# --------------------------------------------------------------------------
def make_cache(k, v, lens, dtype, seed=0, spare=5):
    """Dense k, v [B, L, nKV, hd] -> paged cache with a shuffled page table."""
    B, L, nKV, hd = k.shape
    per = -(-L // PAGE)
    n_pages = B * per + spare
    perm = np.random.default_rng(seed).permutation(n_pages)
    table = torch.zeros(B, per + 2, dtype=torch.int32)
    kc = torch.full((n_pages, nKV, PAGE, hd), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((n_pages, nKV, PAGE, hd), float("nan"), dtype=dtype, device=DEV)
    c = 0
    for b in range(B):
        for p in range(-(-int(lens[b]) // PAGE)):
            page = int(perm[c]); c += 1
            table[b, p] = page
            n = min(PAGE, int(lens[b]) - p * PAGE)
            kc[page, :, :n] = k[b, p * PAGE:p * PAGE + n].transpose(0, 1).to(dtype)
            vc[page, :, :n] = v[b, p * PAGE:p * PAGE + n].transpose(0, 1).to(dtype)
    return kc, vc, table.to(DEV)


def ref_attention(q, k, v, ctx, qlen, window):
    """q [qlen, nH, hd] at positions ctx..ctx+qlen-1 over k, v [ctx+qlen, nKV, hd] (float64)."""
    nH, nKV = q.shape[1], k.shape[1]
    out = torch.zeros_like(q)
    for h in range(nH):
        g = h // (nH // nKV)
        for i in range(qlen):
            p = ctx + i
            lo = max(0, p - window + 1) if window > 0 else 0
            s = k[lo:p + 1, g] @ q[i, h]
            w = torch.softmax(s, 0)
            out[i, h] = (w[:, None] * v[lo:p + 1, g]).sum(0)
    return out


@pytest.mark.parametrize("nH,nKV,hd", [(3, 3, 16), (4, 2, 80), (6, 1, 48), (5, 5, 32), (2, 2, 128), (2, 1, 64), (2, 2, 96), (1, 1, 112)])
@pytest.mark.parametrize("window", [0, 37, 150])
def test_attention_prefill_tc(nH, nKV, hd, window):
    run_attention("prefill_tc", torch.bfloat16, nH, nKV, hd, window, [0, 130, 63, 5, 200], [70, 1, 66, 9, 300])
    assert all(v == 0 for v in ops().wait_failures().values()), "a bounded wait ran out"


@pytest.mark.parametrize("hd,window", [(80, 0), (128, 0), (64, 333)])
def test_attention_prefill_tc_long(hd, window):
    """Many pages: the key and value rings wrap several times, the two tiles of a block end on
    different pages, and a sequence's rows start deep in its context."""
    run_attention("prefill_tc", torch.bfloat16, 2, 1, hd, window, [700, 0, 1111], [1500, 517, 130])
    assert all(v == 0 for v in ops().wait_failures().values()), "a bounded wait ran out"


@pytest.mark.parametrize("nH,nKV,hd", [(3, 3, 16), (4, 2, 80), (6, 1, 48), (2, 2, 256), (5, 5, 32), (2, 2, 128)])
@pytest.mark.parametrize("window", [0, 37, 150])
def test_attention_prefill(nH, nKV, hd, window):
    run_attention("prefill", torch.bfloat16, nH, nKV, hd, window, [0, 130, 63, 5, 200], [70, 1, 66, 9, 300])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nH,nKV,hd", [(3, 3, 16), (4, 2, 80), (6, 1, 48), (2, 2, 256), (5, 5, 40)])
@pytest.mark.parametrize("window", [0, 37])
def test_attention_generic(dtype, nH, nKV, hd, window):
    run_attention("generic", dtype, nH, nKV, hd, window, [0, 130, 63, 5], [70, 1, 66, 9])


def run_attention(kernel, dtype, nH, nKV, hd, window, ctxs, qlens):
    o = ops()
    B, L = len(ctxs), max(c + q for c, q in zip(ctxs, qlens))
    k = rnd(B, L, nKV, hd, seed=1).to(dtype).float()
    v = rnd(B, L, nKV, hd, seed=2).to(dtype).float()
    lens = [c + q for c, q in zip(ctxs, qlens)]
    kc, vc, table = make_cache(k, v, lens, dtype)
    T = sum(qlens)
    q = (rnd(T, nH, hd, seed=3) / math.sqrt(hd)).to(dtype)
    out = torch.empty(T, nH * hd, dtype=dtype, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    starts = np.concatenate([[0], np.cumsum(qlens)[:-1]]).tolist()
    fn = {"generic": o.attention_generic, "prefill": o.attention_prefill, "prefill_tc": o.attention_prefill_tc}[kernel]
    fn(q.reshape(T, nH * hd), out, kc, vc, i32(starts), i32(qlens), i32(ctxs), table,
       nH, nKV, hd, max(qlens), window)
    tol = 2e-5 if dtype == torch.float32 else 2 ** -7
    for b in range(B):
        ref = ref_attention(q[starts[b]:starts[b] + qlens[b]].double().cpu(), k[b, :lens[b]].double().cpu(),
                            v[b, :lens[b]].double().cpu(), ctxs[b], qlens[b], window)
        got = out[starts[b]:starts[b] + qlens[b]].reshape(qlens[b], nH, hd).double().cpu()
        assert torch.isfinite(got).all()
        assert (got - ref).abs().max() <= tol * max(1.0, ref.abs().max().item()), (b,)


@pytest.mark.parametrize("nH,nKV,hd", [(4, 4, 16), (4, 2, 80), (6, 2, 48), (8, 1, 64), (2, 2, 256), (3, 3, 32)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode(nH, nKV, hd, window):
    o = ops()
    ctxs = [0, 63, 64, 700, 1, 333]
    B, L = len(ctxs), max(ctxs) + 1
    dtype = torch.bfloat16
    k = rnd(B, L, nKV, hd, seed=1).to(dtype).float()
    v = rnd(B, L, nKV, hd, seed=2).to(dtype).float()
    lens = [c + 1 for c in ctxs]
    kc, vc, table = make_cache(k, v, lens, dtype, seed=3)
    q = (rnd(B, nH, hd, seed=3) / math.sqrt(hd)).to(dtype)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    for splits, scratch in ((1, None), (2, None), (5, None), (8, None), (16, None), (3, torch.empty(B * nH * 3 * (hd + 2), device=DEV))):
        out = torch.empty(B, nH * hd, dtype=dtype, device=DEV)
        o.attention_decode(q.reshape(B, nH * hd), out, kc, vc, i32(ctxs), table, nH, nKV, hd, splits, window,
                           scratch=scratch)
        for b in range(B):
            ref = ref_attention(q[b:b + 1].double().cpu(), k[b, :lens[b]].double().cpu(),
                                v[b, :lens[b]].double().cpu(), ctxs[b], 1, window)
            got = out[b].reshape(1, nH, hd).double().cpu()
            assert torch.isfinite(got).all()
            assert (got - ref).abs().max() <= 2 ** -7 * max(1.0, ref.abs().max().item()), (b, splits)


@pytest.mark.parametrize("nH,nKV,hd,rot", [(4, 4, 16, 16), (4, 2, 80, 32), (6, 2, 48, 0), (8, 1, 64, 16), (2, 2, 256, 64), (3, 3, 32, 32)])
@pytest.mark.parametrize("window", [0, 100])
def test_attention_decode_from_the_projection(nH, nKV, hd, rot, window):
    """Decode attention that takes the projection's output (rotating and scaling the queries, storing the
    new key and value itself) against the separate kernel followed by decode attention: the same output
    bit for bit and the same cache, at the new positions and everywhere else."""
    o = ops()
    ctxs = [0, 63, 64, 700, 1, 333]
    B, L = len(ctxs), max(ctxs) + 1
    dtype = torch.bfloat16
    k = rnd(B, L, nKV, hd, seed=1).to(dtype).float()
    v = rnd(B, L, nKV, hd, seed=2).to(dtype).float()
    lens = [c + 1 for c in ctxs]
    kc0, vc0, table = make_cache(k, v, lens, dtype, seed=3)
    i32 = lambda x: torch.tensor(np.asarray(x), dtype=torch.int32, device=DEV)
    qkv = rnd(B, (nH + 2 * nKV) * hd, seed=4).to(dtype)
    cos = sin = None
    if rot:
        from gopherllm_b200.parts.position import rope_inverse_frequencies
        cos, sin = o.rope_table(i32(ctxs), torch.from_numpy(rope_inverse_frequencies(rot, 10000.0)).to(DEV))
    scale = 1.0 / math.sqrt(hd)
    for write_kv in (True, False):
        for splits in (1, 2, 5, 8, 16):
            kc_a, vc_a, kc_b, vc_b = kc0.clone(), vc0.clone(), kc0.clone(), vc0.clone()
            q = torch.empty(B, nH * hd, dtype=dtype, device=DEV)
            o.qkv_to_cache(qkv, q, kc_a, vc_a, i32(np.arange(B)), i32(ctxs), table, nH, nKV, hd, scale, cos, sin,
                           write_kv=write_kv)
            want = torch.empty(B, nH * hd, dtype=dtype, device=DEV)
            o.attention_decode(q, want, kc_a, vc_a, i32(ctxs), table, nH, nKV, hd, splits, window)
            got = torch.empty_like(want)
            o.attention_decode(None, got, kc_b, vc_b, i32(ctxs), table, nH, nKV, hd, splits, window,
                               qkv=qkv, cos=cos, sin=sin, q_scale=scale, write_kv=write_kv)
            torch.cuda.synchronize()
            same = lambda x, y: torch.equal(x.view(torch.int16), y.view(torch.int16))      # unused cells are NaN
            assert same(kc_a, kc_b) and same(vc_a, vc_b), (write_kv, splits)
            assert torch.equal(got, want), (write_kv, splits, (got.float() - want.float()).abs().max().item())


@pytest.mark.parametrize("kernel", ["generic32", "generic16", "decode", "prefill", "prefill_tc"])
def test_attention_far_key_and_window_edge(kernel):
    """One key among hundreds carries the whole weight: its value must come back.  With a
    window the key at the window's edge is seen and the one before it is not."""
    o = ops()
    nH = nKV = 2
    hd, L = 32, 600
    dtype = torch.float32 if kernel == "generic32" else torch.bfloat16
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    for far, window, seen in [(3, 0, True), (64, 0, True), (599 - 99, 100, True), (599 - 100, 100, False),
                              (599, 1, True), (598, 1, False), (0, 600, True), (0, 599, False)]:
        k = torch.zeros(1, L, nKV, hd)
        v = rnd(1, L, nKV, hd, seed=9).cpu()
        k[0, far, :, 0] = 50.0                       # score 50 for this key, 0 for all others
        q = torch.zeros(1, nH, hd)
        q[..., 0] = 1.0
        kc, vc, table = make_cache(k.to(DEV), v.to(DEV), [L], dtype, seed=far)
        out = torch.empty(1, nH * hd, dtype=dtype, device=DEV)
        qd = q.reshape(1, nH * hd).to(dtype).to(DEV)
        if kernel == "decode":
            o.attention_decode(qd, out, kc, vc, i32([L - 1]), table, nH, nKV, hd, 3, window)
        elif kernel == "prefill":
            o.attention_prefill(qd, out, kc, vc, i32([0]), i32([1]), i32([L - 1]), table, nH, nKV, hd, 1, window)
        elif kernel == "prefill_tc":
            o.attention_prefill_tc(qd, out, kc, vc, i32([0]), i32([1]), i32([L - 1]), table, nH, nKV, hd, 1, window)
        else:
            o.attention_generic(qd, out, kc, vc, i32([0]), i32([1]), i32([L - 1]), table, nH, nKV, hd, 1, window)
        got = out.reshape(nH, hd).float().cpu()
        want = v[0, far].to(dtype).float()
        hit = (got - want).abs().max().item() < 0.02
        assert hit == seen, (far, window, seen, (got - want).abs().max().item())


# --------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nH,nKV,hd,rot", [(4, 4, 16, 8), (6, 2, 48, 24), (2, 2, 80, 32), (3, 1, 32, 0), (2, 2, 64, 64)])
@pytest.mark.parametrize("qk_norm", [False, True])
def test_qkv_to_cache(dtype, nH, nKV, hd, rot, qk_norm):
    o = ops()
    ctxs, qlens = [0, 100, 63], [66, 1, 2]
    B, T = len(ctxs), sum(qlens)
    theta, eps, scale = 500000.0, 1e-6, 1.0 / math.sqrt(hd)
    tok_seq = np.repeat(np.arange(B), qlens)
    tok_pos = np.concatenate([np.arange(c, c + n) for c, n in zip(ctxs, qlens)])
    qkv = rnd(T, (nH + 2 * nKV) * hd, seed=4).to(dtype)
    per = 3
    table = torch.tensor(np.random.default_rng(1).permutation(B * per).reshape(B, per), dtype=torch.int32, device=DEV)
    kc = torch.zeros(B * per, nKV, PAGE, hd, dtype=dtype, device=DEV)
    vc = torch.zeros_like(kc)
    i32 = lambda x: torch.tensor(np.asarray(x), dtype=torch.int32, device=DEV)
    cos = sin = None
    if rot:
        from gopherllm_b200.parts.position import rope_inverse_frequencies
        inv = rope_inverse_frequencies(rot, theta)
        assert np.array_equal(inv, plain_phi.rope_inv_freq(rot, theta))
        cos, sin = o.rope_table(i32(tok_pos), torch.from_numpy(inv).to(DEV))
        rs, rc = plain_phi.rope_tables(tok_pos, rot, theta)
        assert (cos.cpu() - rc).abs().max() <= 2e-7 and (sin.cpu() - rs).abs().max() <= 2e-7
    norms = None
    if qk_norm:
        norms = [(rnd(hd, seed=5) + 1.0, rnd(hd, seed=6)), (rnd(hd, seed=7) + 1.0, rnd(hd, seed=8))]
    q_out = torch.empty(T, nH * hd, dtype=dtype, device=DEV)
    o.qkv_to_cache(qkv, q_out, kc, vc, i32(tok_seq), i32(tok_pos), table, nH, nKV, hd, scale, cos, sin,
                   q_norm=norms[0] if norms else None, k_norm=norms[1] if norms else None, norm_eps=eps)
    x = qkv.double().cpu().reshape(T, nH + 2 * nKV, hd)
    q, k, v = x[:, :nH], x[:, nH:nH + nKV], x[:, nH + nKV:]
    if qk_norm:
        q = plain_phi.layer_norm(q, norms[0][0].double().cpu(), norms[0][1].double().cpu(), eps)
        k = plain_phi.layer_norm(k, norms[1][0].double().cpu(), norms[1][1].double().cpu(), eps)
    if rot:
        rs, rc = plain_phi.rope_tables(tok_pos, rot, theta)
        q, k = plain_phi.apply_rope(q, rs, rc, rot), plain_phi.apply_rope(k, rs, rc, rot)
    q = q * scale
    tol = 1e-5 if dtype == torch.float32 else 2 ** -7
    assert (q_out.double().cpu().reshape(T, nH, hd) - q).abs().max() <= tol * max(1.0, q.abs().max().item())
    for t in range(T):
        page = int(table[tok_seq[t], tok_pos[t] // PAGE])
        gk = kc[page, :, tok_pos[t] % PAGE].double().cpu()
        gv = vc[page, :, tok_pos[t] % PAGE].double().cpu()
        assert (gk - k[t]).abs().max() <= tol * max(1.0, k.abs().max().item()), t
        assert torch.equal(gv, v[t].to(dtype).double()), t
    if rot and rot < hd and not qk_norm:       # dims past the rotary part pass through untouched
        want = (x[:, :nH, rot:].float() * torch.tensor(scale, dtype=torch.float32)).to(dtype)
        assert torch.equal(q_out.reshape(T, nH, hd)[..., rot:].cpu(), want)
        got = torch.stack([kc[int(table[tok_seq[t], tok_pos[t] // PAGE]), :, tok_pos[t] % PAGE, rot:] for t in range(T)])
        assert torch.equal(got.double().cpu(), x[:, nH:nH + nKV, rot:].to(dtype).double())
    written = sum(qlens) * nKV * hd
    assert int((kc != 0).sum()) <= written      # nothing outside the steps' positions was touched


# --------------------------------------------------------------------------
@pytest.mark.parametrize("V", [50, 1000, 51200])
def test_sampling_matches_plain(V):
    o = ops()
    B = 5
    rng = np.random.default_rng(V)
    logits = (rng.standard_normal((B, V)) * 3).astype(np.float32)
    logits[1, 7] = np.nan
    logits[2, 3] = np.inf
    logits[3, : V // 2] = logits[3, V // 2 - 1]          # many equal values
    if V >= 1000:                                        # one token far above a flat rest: the rest's weights fall
        logits[4] = (rng.standard_normal(V) * 0.01).astype(np.float32)     # under 1e-5 of the best, yet carry mass
        logits[4, 17] = 12.0
    recents = [list(rng.integers(0, V, size=n)) for n in (0, 5, 64, 64, 30)]
    recents[2][5] = recents[2][9]                        # a token twice in the window
    cases = [dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0),
             dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.3),
             dict(temperature=0.7, top_k=40, top_p=0.9, min_p=0.0, repeat_penalty=1.1),
             dict(temperature=0.95, top_k=7, top_p=0.95, min_p=0.05, repeat_penalty=1.05),
             dict(temperature=1.5, top_k=1, top_p=0.9, min_p=0.0, repeat_penalty=1.0),
             dict(temperature=0.8, top_k=33, top_p=1.0, min_p=0.0, repeat_penalty=1.0),
             dict(temperature=0.8, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0),
             dict(temperature=1.0, top_k=V + 5, top_p=1.0, min_p=0.0, repeat_penalty=1.2),
             # the nucleus over the whole row (top-k off): sorted candidates, min-p and top-p cuts
             dict(temperature=0.7, top_k=0, top_p=0.9, min_p=0.0, repeat_penalty=1.1),
             dict(temperature=1.3, top_k=0, top_p=0.5, min_p=0.1, repeat_penalty=1.0),
             dict(temperature=0.4, top_k=0, top_p=1.0, min_p=0.3, repeat_penalty=1.0),
             dict(temperature=5.0, top_k=V, top_p=0.97, min_p=0.0, repeat_penalty=1.0),
             dict(temperature=1.0, top_k=0, top_p=0.999, min_p=0.0, repeat_penalty=1.0),
             dict(temperature=2.5, top_k=0, top_p=0.3, min_p=0.0, repeat_penalty=1.0),
             dict(temperature=1.0, top_k=0, top_p=1.0, min_p=0.02, repeat_penalty=1.15)]
    for ci, c in enumerate(cases):
        if c["top_k"] > 0 and c["top_k"] >= V and (c["top_p"] < 1 or c["min_p"] > 0):
            continue
        dl = torch.from_numpy(logits).to(DEV)
        work = torch.empty(B, V, device=DEV)
        recent = torch.zeros(B, 64, dtype=torch.int32)
        for i, r in enumerate(recents):
            recent[i, :len(r)] = torch.tensor(r, dtype=torch.int32)
        recent = recent.to(DEV)
        recent_n = torch.tensor([len(r) for r in recents], dtype=torch.int32, device=DEV)
        seeds = [11 + ci, 0xDEADBEEFCAFE1337, 3, 2 ** 63 + 5, 99]
        rng_state = torch.tensor([s - 2 ** 64 if s >= 2 ** 63 else s for s in seeds], dtype=torch.int64, device=DEV)
        out = torch.zeros(B, dtype=torch.int32, device=DEV)
        draws = 6 if c["top_k"] == 0 else 3
        got = []
        for _ in range(draws):
            o.sample(dl, work, recent, recent_n, rng_state, out, **c)
            got.append(out.cpu().tolist())
        assert torch.equal(dl.cpu().nan_to_num(0, 0, 0), torch.from_numpy(logits).nan_to_num(0, 0, 0)), "logits were modified"
        for i in range(B):
            r = plain_phi.Rng(seeds[i])
            rec = list(recents[i])
            for d in range(draws):
                state_before = r.state
                want = plain_phi.sample(logits[i], c["temperature"], c["top_k"], c["top_p"], c["min_p"],
                                        c["repeat_penalty"], r, rec)
                whole_row = c["temperature"] >= 1e-6 and not (0 < c["top_k"] < V)
                nucleus = whole_row and (c["top_p"] < 1 or c["min_p"] > 0)
                if whole_row and not nucleus and got[d][i] != want:
                    # The whole-row draw walks a running 32-bit sum of V weights; the plain loop adds
                    # them one by one, the kernel by a parallel scan.  Two such sums of n terms with
                    # total 1 differ by at most n * 2^-24, so the draw u may fall on either side of a
                    # boundary that close: the kernel's token must hold u within that distance.
                    u = float(plain_phi.Rng(state_before).next_f32())
                    lg = logits[i].astype(np.float64).copy()
                    lg[~np.isfinite(lg)] = -np.inf
                    pen = np.float64(np.float32(c["repeat_penalty"]))
                    for tok in rec:
                        if lg[tok] > -np.inf and pen != 1:
                            lg[tok] = lg[tok] / pen if lg[tok] > 0 else lg[tok] * pen
                    wts = np.exp((lg - lg.max()) / np.float64(np.float32(c["temperature"])))
                    cdf = np.cumsum(wts / wts.sum())
                    g_ = got[d][i]
                    slack = V * 2.0 ** -24
                    lo_edge = cdf[g_ - 1] if g_ > 0 else 0.0
                    assert lo_edge - slack <= u <= cdf[g_] + slack, (ci, i, d, g_, want, u, lo_edge, cdf[g_])
                    want = g_
                if nucleus and got[d][i] != want:
                    # The reference walks running 32-bit sums over the sorted candidates, one by one; the
                    # kernel adds mass exactly (fixed point).  Over thousands of candidates the two differ
                    # by up to n * 2^-24 of the total, more than a tail candidate's weight, so the cut and
                    # the draw may fall a few candidates apart.  The kernel's token must then be right for
                    # the exact sums: inside the exact cut (give or take that slack), with the draw u * kept
                    # inside its interval of the exact running mass, give or take the same.
                    u = float(plain_phi.Rng(state_before).next_f32())
                    lg = logits[i].astype(np.float32).copy()
                    lg[~np.isfinite(lg)] = -np.inf
                    pen = np.float32(c["repeat_penalty"])
                    for tok in rec:
                        if lg[tok] > -np.inf and pen != 1:
                            lg[tok] = lg[tok] / pen if lg[tok] > 0 else lg[tok] * pen
                    inv_t = np.float32(1.0) / np.float32(c["temperature"])
                    wts = np.exp(((lg - lg.max()) * inv_t).astype(np.float64)).astype(np.float32).astype(np.float64)
                    total = wts.sum()
                    thr = np.float64(np.float32(wts.max()) * np.float32(1e-5))
                    cand = np.nonzero(wts >= thr)[0]
                    if wts[cand].sum() < np.float64(np.float32(c["top_p"])) * total:
                        cand = np.arange(V)
                    order = cand[np.lexsort((cand, -wts[cand]))]
                    sw = wts[order]
                    n_c = len(order)
                    if c["min_p"] > 0:
                        keep = sw >= np.float64(np.float32(c["min_p"]) * np.float32(sw[0]))
                        n_c = int(keep.sum())
                        total = sw[:n_c].sum()
                    cs = np.cumsum(sw[:n_c])
                    slack = n_c * 2.0 ** -24 * total
                    target = np.float64(np.float32(c["top_p"])) * total
                    over = np.nonzero(cs > target + slack)[0]
                    cut_hi = int(over[0]) + 1 if len(over) else n_c            # the cut is at most here ...
                    over = np.nonzero(cs > target - slack)[0]
                    cut_lo = int(over[0]) + 1 if len(over) else n_c            # ... and at least here
                    g_ = got[d][i]
                    pos = int(np.nonzero(order[:n_c] == g_)[0][0]) if g_ in order[:n_c] else -1
                    assert 0 <= pos < cut_hi, (ci, i, d, g_, want, pos, cut_lo, cut_hi)
                    lo_edge = cs[pos - 1] if pos > 0 else 0.0
                    ok = any(lo_edge - slack <= u * cs[cut - 1] <= cs[pos] + slack for cut in {cut_lo, cut_hi})
                    assert ok or pos == cut_hi - 1, (ci, i, d, g_, want, pos, u, lo_edge, cs[pos], cs[cut_lo - 1], cs[cut_hi - 1])
                    want = g_
                assert got[d][i] == want, (ci, i, d, got[d][i], want)
                rec = (rec + [want])[-64:]


# --------------------------------------------------------------------------
# the fused decode layer: one kernel for norm, both branches and the residual sum
# --------------------------------------------------------------------------
@pytest.mark.parametrize("M,nH,nKV,hd,D,I,rot,window,rms,act,bias", [
    (5, 4, 4, 64, 256, 328, 32, 0, False, "gelu_new", True),      # a page's edge, an empty cache, several pages
    (40, 8, 2, 32, 264, 520, 16, 100, True, "relu", False),       # grouped heads, a window, no biases, 40 tokens
    (64, 2, 1, 128, 256, 256, 0, 0, False, "gelu", True),         # the largest head and batch, no rotation
    (17, 6, 3, 48, 288, 200, 48, 0, False, "gelu_new", True),     # head size 48, a fully rotated head
    (1, 32, 32, 80, 2560, 10240, 32, 0, False, "gelu_new", True), # one token at Phi-2's sizes
    (64, 32, 32, 80, 2560, 10240, 32, 0, False, "gelu_new", True),  # 64 tokens at Phi-2's sizes: whole tiles to a block, seven blocks a tile in the last product
    (24, 8, 8, 80, 1032, 4104, 32, 0, False, "gelu_new", True),   # 24 tokens (padded to 32), widths that end inside a chunk
])
def test_decode_layer(M, nH, nKV, hd, D, I, rot, window, rms, act, bias):
    """norm -> (attention over the paged cache | feed-forward) -> residual sum as one kernel, against the
    same layer written out in 64-bit: the residual stream, and the cache (the new token's rotated key and
    its value where they belong, everything else, NaN filling included, untouched)."""
    o = ops()
    rng = np.random.default_rng(M + hd)
    ctxs = [0, 63, 64, 200, 129][:M] if M <= 5 else [int(c) for c in rng.integers(0, 300, size=M)]
    dtype = torch.bfloat16
    L = max(ctxs) + 1
    k = rnd(M, L, nKV, hd, seed=1).to(dtype).float()
    v = rnd(M, L, nKV, hd, seed=2).to(dtype).float()
    kc, vc, table = make_cache(k, v, [c + 1 for c in ctxs], dtype, seed=3)
    for b, c in enumerate(ctxs):                               # the new token's row is not there yet
        page = int(table[b, c // PAGE])
        kc[page, :, c % PAGE] = float("nan")
        vc[page, :, c % PAGE] = float("nan")
    kc0, vc0 = kc.clone(), vc.clone()
    i32 = lambda t: torch.tensor(np.asarray(t), dtype=torch.int32, device=DEV)
    Nqkv, No = (nH + 2 * nKV) * hd, nH * hd
    x = rnd(M, D, seed=4)
    g, b_ = 1 + rnd(D, scale=0.1, seed=5), (rnd(D, scale=0.1, seed=6) if not rms else None)
    s = 1.0 / math.sqrt(D)
    w_qkv, w_up = rnd(Nqkv, D, scale=s, seed=7).to(dtype), rnd(I, D, scale=s, seed=8).to(dtype)
    w_out, w_down = rnd(D, No, scale=1 / math.sqrt(No), seed=9).to(dtype), rnd(D, I, scale=1 / math.sqrt(I), seed=10).to(dtype)
    bq, bu, bo, bd = ((rnd(n, scale=0.1, seed=11 + i) for i, n in enumerate((Nqkv, I, D, D))) if bias else (None,) * 4)
    cos = sin = None
    if rot:
        from gopherllm_b200.parts.position import rope_inverse_frequencies
        cos, sin = o.rope_table(i32(ctxs), torch.from_numpy(rope_inverse_frequencies(rot, 10000.0)).to(DEV))
    scale = 1.0 / math.sqrt(hd)
    x0 = x.clone()
    o.decode_layer(x, g, b_, 1e-5, rms, w_qkv, bq, w_up, bu, act, w_out, bo, w_down, bd, kc, vc, i32(ctxs), table,
                   nH, nKV, hd, scale, cos, sin, window, True)
    torch.cuda.synchronize()
    assert all(val == 0 for val in o.wait_failures().values()), "a bounded wait ran out"
    # the same layer in 64-bit, rounding to bfloat16 where the kernel's buffers do
    r16 = lambda t: t.to(dtype).double()
    xd = x0.double().cpu()
    if rms:
        n = xd / torch.sqrt((xd * xd).mean(-1, keepdim=True) + 1e-5) * g.double().cpu()
    else:
        n = plain_phi.layer_norm(xd, g.double().cpu(), b_.double().cpu(), 1e-5)
    n = r16(n)
    z = lambda t, m: t.double().cpu() if t is not None else torch.zeros(m, dtype=torch.float64)
    qkv = r16(n @ w_qkv.double().cpu().T + z(bq, Nqkv))
    h = r16(gelu_ref(n @ w_up.double().cpu().T + z(bu, I), act))
    q, kn, vn = qkv[:, :No].reshape(M, nH, hd), qkv[:, No:No + nKV * hd].reshape(M, nKV, hd), qkv[:, No + nKV * hd:].reshape(M, nKV, hd)
    if rot:
        q = plain_phi.apply_rope(q, sin.double().cpu(), cos.double().cpu(), rot)
        kn = plain_phi.apply_rope(kn, sin.double().cpu(), cos.double().cpu(), rot)
    q, kn = r16(q * scale), r16(kn)
    att = torch.zeros(M, nH, hd, dtype=torch.float64)
    for b, c in enumerate(ctxs):
        kk = torch.cat([k[b, :c].double().cpu(), kn[b:b + 1]])
        vv = torch.cat([v[b, :c].double().cpu(), vn[b:b + 1]])
        att[b] = ref_attention(q[b:b + 1], kk, vv, c, 1, window)[0]
    att = r16(att.reshape(M, No))
    want = xd + att @ w_out.double().cpu().T + z(bo, D) + h @ w_down.double().cpu().T + z(bd, D)
    got = x.double().cpu()
    assert torch.isfinite(got).all()
    err = (got - want).abs().max().item()
    assert err <= 2 ** -6 * max(1.0, (want - xd).abs().max().item()), (err, (want - xd).abs().max().item())
    # the cache: the new rows, and nothing else
    for b, c in enumerate(ctxs):
        page = int(table[b, c // PAGE])
        assert (kc[page, :, c % PAGE].double().cpu() - kn[b]).abs().max() <= 2 ** -7 * max(1.0, kn[b].abs().max().item()), b
        assert (vc[page, :, c % PAGE].double().cpu() - vn[b]).abs().max() <= 2 ** -7 * max(1.0, vn[b].abs().max().item()), b
        kc0[page, :, c % PAGE] = kc[page, :, c % PAGE]
        vc0[page, :, c % PAGE] = vc[page, :, c % PAGE]
    same = lambda a_, b2: torch.equal(a_.view(torch.int16), b2.view(torch.int16))
    assert same(kc, kc0) and same(vc, vc0), "the kernel wrote to the cache outside the new tokens' rows"
