"""The tape of launches that lets a model repeat one block's launches for the next equal block: what it
takes for two tapes to count as the same launches, and what a repeat substitutes (no device needed: the
"kernels" are Python callables that note what they were called with)."""
import ctypes
from ctypes import Structure, byref, c_float, c_int, c_void_p

import torch

from gopherllm_b200 import ops


class Args(Structure):
    _fields_ = [("a", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("M", c_int), ("scale", c_float)]


class Fake:
    """Stands in for a library's launcher: notes the values it was called with, returns 0."""

    def __init__(self):
        self.calls = []

    def __call__(self, *args):
        seen = []
        for x in args:
            st = getattr(x, "_obj", None)
            if isinstance(st, Structure):
                seen.append(tuple(getattr(st, n) for n, _ in st._fields_))
            else:
                seen.append(x.value)
        self.calls.append(tuple(seen))
        return 0


def record(fn_gemm, fn_norm, w, bias, gamma, act, m=8, scale=0.5, temp=None):
    """One "block": a norm and a product, as ops' functions would launch them."""
    tape = ops.LaunchTape().start()
    try:
        if temp is not None:
            tape.temps.append(temp)
        t = temp.data_ptr() if temp is not None else 0x9000
        ops._check(ops._launch(fn_norm, c_void_p(act), c_void_p(gamma), c_void_p(t), c_int(m), ops._StreamArg(7)), "norm")
        a = Args(t, w, bias, m, scale)
        ops._check(ops._launch(fn_gemm, byref(a), c_int(3), ops._StreamArg(7)), "gemm")
    finally:
        tape.stop()
    return tape


def test_same_launches_but_for_the_blocks_own_tensors():
    g, n = Fake(), Fake()
    one = dict(w=0x1000, bias=0x1100, gamma=0x1200)
    two = dict(w=0x2000, bias=0x2100, gamma=0x2200)
    t1 = record(g, n, one["w"], one["bias"], one["gamma"], act=0x5000)
    t2 = record(g, n, two["w"], two["bias"], two["gamma"], act=0x5000)
    assert t1.same_as(t2, one, two)
    assert not t1.same_as(t2, one, dict(two, w=0x2008))            # a tensor of the second block that the tape does not show
    assert not t1.same_as(record(g, n, two["w"], two["bias"], two["gamma"], act=0x5000, m=9), one, two)      # a size
    assert not t1.same_as(record(g, n, two["w"], two["bias"], two["gamma"], act=0x5000, scale=0.25), one, two)
    assert not t1.same_as(record(g, n, two["w"], two["bias"], two["gamma"], act=0x5008), one, two)          # a shared input moved
    assert not t1.same_as(record(Fake(), n, two["w"], two["bias"], two["gamma"], act=0x5000), one, two)     # another kernel
    assert not t1.same_as(record(g, n, two["w"], None, two["gamma"], act=0x5000), one, dict(two, bias=0))   # a bias that is not there
    # a pointer into a tensor (not its start) is not substituted, so the tapes differ: such a block is never repeated
    t3 = record(g, n, one["w"] + 64, one["bias"], one["gamma"], act=0x5000)
    t4 = record(g, n, two["w"] + 64, two["bias"], two["gamma"], act=0x5000)
    assert not t3.same_as(t4, one, two)


def test_temporaries_pair_up_in_order_and_a_repeat_uses_the_recorded_ones(monkeypatch):
    monkeypatch.setattr(ops, "_stream", lambda: ops._StreamArg(11))     # (no device here: the current stream is a number)
    g, n = Fake(), Fake()
    one = dict(w=0x1000, bias=0x1100, gamma=0x1200)
    two = dict(w=0x2000, bias=0x2100, gamma=0x2200)
    three = dict(w=0x3000, bias=0, gamma=0x3200)
    x1, x2 = torch.empty(16), torch.empty(16)
    t1 = record(g, n, one["w"], one["bias"], one["gamma"], act=0x5000, temp=x1)
    t2 = record(g, n, two["w"], two["bias"], two["gamma"], act=0x5000, temp=x2)
    assert t1.same_as(t2, one, two)
    assert not t1.same_as(record(g, n, two["w"], two["bias"], two["gamma"], act=0x5000, temp=torch.empty(17)), one, two)
    t1.bind(one)
    g.calls.clear()
    n.calls.clear()
    before = ops.LAUNCHES
    t1.repeat(three)
    assert ops.LAUNCHES == before + 2
    assert n.calls[-1] == (0x5000, 0x3200, x1.data_ptr(), 8, 11)       # the third block's gamma, the recorded temporary, the stream current now
    assert g.calls[-1][0] == (x1.data_ptr(), 0x3000, None, 8, 0.5)      # its weight; no bias: a null pointer
    t1.repeat(two)
    assert g.calls[-1][0][:3] == (x1.data_ptr(), 0x2000, 0x2100)


def test_a_tape_is_not_recorded_inside_another():
    t = ops.LaunchTape().start()
    try:
        try:
            ops.LaunchTape().start()
            raise AssertionError("a second tape started")
        except ops.KernelError:
            pass
    finally:
        t.stop()
    assert ops._TAPE is None
