"""gl_attention_decode_static: the decode attention entry point that allocates nothing.

Some hosts of this library cannot obtain device memory while they run (all of it was
handed to their own pools at start-up, or an allocation's device-wide synchronisation is
not acceptable, or they are plain C programs without PyTorch's allocator).  For them the
library exports a variant of decode attention whose scratch for the split partial results
is an array built into the library.  This test calls it the way such a host would, through
the exported C symbol, and checks it against the ordinary entry point, whose scratch the
caller provides.  It runs last so that a failure here cannot hide any other test.
"""
import ctypes
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
PAGE = 64


class DecodeArgs(ctypes.Structure):
    """The launcher's argument record (DecodeArgs in csrc/attention_decode.cu)."""
    _fields_ = [("q", ctypes.c_void_p), ("out", ctypes.c_void_p), ("k_cache", ctypes.c_void_p),
                ("v_cache", ctypes.c_void_p), ("seq_ctx", ctypes.c_void_p), ("pages", ctypes.c_void_p),
                ("part_o", ctypes.c_void_p), ("part_ml", ctypes.c_void_p),
                ("B", ctypes.c_int), ("nH", ctypes.c_int), ("nKV", ctypes.c_int), ("max_pages", ctypes.c_int),
                ("window", ctypes.c_int), ("splits", ctypes.c_int)]


def library(head_dim):
    """The shared library itself, opened with ctypes as a C host would open it."""
    from gopherllm_b200.csrc import build, catalog
    lib = ctypes.CDLL(build.library_path("attention_decode.cu", catalog.head_dim_defines(head_dim)))
    lib.gl_attention_decode_static.restype = ctypes.c_int
    lib.gl_attention_decode_static.argtypes = [ctypes.POINTER(DecodeArgs), ctypes.c_void_p]
    lib.gl_attention_decode_static_capacity.restype = ctypes.c_longlong
    lib.gl_attention_decode_scratch.restype = ctypes.c_longlong
    return lib


@pytest.mark.parametrize("nH,nKV,hd,splits", [(8, 8, 80, 4), (6, 2, 48, 3)])
def test_static_scratch_matches_caller_scratch_twice_in_a_row(nH, nKV, hd, splits):
    from gopherllm_b200 import ops
    lib = library(hd)
    g = torch.Generator().manual_seed(7)
    ctxs = [0, 63, 64, 500, 333]
    B, n_pages_seq = len(ctxs), max(ctxs) // PAGE + 1
    n_pages = B * n_pages_seq + 3
    kc = torch.randn(n_pages, nKV, PAGE, hd, generator=g).to(torch.bfloat16).to(DEV)
    vc = torch.randn(n_pages, nKV, PAGE, hd, generator=g).to(torch.bfloat16).to(DEV)
    perm = np.random.default_rng(1).permutation(n_pages)[: B * n_pages_seq].reshape(B, n_pages_seq)
    pages = torch.tensor(perm, dtype=torch.int32, device=DEV)
    seq_ctx = torch.tensor(ctxs, dtype=torch.int32, device=DEV)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.gl_attention_decode_scratch(B, nH, splits) <= lib.gl_attention_decode_static_capacity()
    for call in range(2):                              # the second call finds the first one's leftovers
        q = (torch.randn(B, nH * hd, generator=g) / math.sqrt(hd)).to(torch.bfloat16).to(DEV)
        want = torch.empty_like(q)
        ops.attention_decode(q, want, kc, vc, seq_ctx, pages, nH, nKV, hd, splits)      # caller's scratch
        got = torch.full_like(q, float("nan"))
        args = DecodeArgs(q.data_ptr(), got.data_ptr(), kc.data_ptr(), vc.data_ptr(), seq_ctx.data_ptr(),
                          pages.data_ptr(), None, None, B, nH, nKV, pages.shape[1], 0, splits)
        if call == 0:
            # the very first call loads the kernels' module and looks the array's address up: once
            # that is done, a call must leave the device's free memory as it found it
            assert lib.gl_attention_decode_static(ctypes.byref(args), stream) == 0
            torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        unchanged = False
        for _ in range(3):            # (the device's free memory is everybody's: ask again if it moved)
            free_before, _ = torch.cuda.mem_get_info()
            rc = lib.gl_attention_decode_static(ctypes.byref(args), stream)
            assert rc == 0, f"call {call}: error {rc}"
            torch.cuda.synchronize()
            free_after, _ = torch.cuda.mem_get_info()
            unchanged = unchanged or free_after == free_before
        assert torch.cuda.memory_allocated() == before      # nothing from PyTorch's allocator
        assert unchanged                                    # and nothing from the CUDA runtime behind its back
        assert torch.isfinite(got.float()).all()
        err = (got.float() - want.float()).abs().max().item()
        assert err <= 2 ** -7 * max(1.0, want.float().abs().max().item()), (call, err)


def test_static_scratch_rejects_what_does_not_fit():
    lib = library(80)
    cap = lib.gl_attention_decode_static_capacity()
    B, nH, splits = 64, 32, 8
    assert lib.gl_attention_decode_scratch(B, nH, splits) > cap
    args = DecodeArgs(None, None, None, None, None, None, None, None, B, nH, nH, 32, 0, splits)
    assert lib.gl_attention_decode_static(ctypes.byref(args), None) == -7      # GL_ERR_SCRATCH, nothing launched
    torch.cuda.synchronize()
