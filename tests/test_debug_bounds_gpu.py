"""The build that checks indices inside the kernels (GOPHERLLM_DEBUG_BOUNDS=1), in a process of its own."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import sys
sys.path.insert(0, sys.argv[1])
import torch
from gopherllm_b200 import ops
assert ops.DEBUG_BOUNDS
dev = "cuda:0"
table = torch.randn(50, 16, device=dev).to(torch.bfloat16)
good = ops.embed(table, torch.tensor([0, 49, 7], dtype=torch.int32, device=dev))
torch.cuda.synchronize()
assert ops.bounds_status() == {}, ops.bounds_status()
ops.check_wait_failures()                                   # nothing on record: no error
# a token id past the table: the kernel must not read there (it reads row 0... clamped) and must say so
bad = ops.embed(table, torch.tensor([3, 55, -2], dtype=torch.int32, device=dev))
torch.cuda.synchronize()
st = ops.bounds_status()
assert len(st) == 1, st
kind, value, limit, count = next(iter(st.values()))
assert kind == "token id" and value in (55, -2) and limit == 50 and count >= 2, st   # (every thread that met it counts)
assert torch.isfinite(bad.float()).all() and torch.equal(bad[0], good[0] * 0 + table[3].float())
try:
    ops.check_wait_failures()
except ops.KernelError as e:
    assert "token id" in str(e) and "limit 50" in str(e), str(e)
else:
    raise AssertionError("a bad index on record raised nothing")
assert ops.bounds_status() == {}                            # cleared by the check
# a page number past the cache: the write goes to page 0 and is reported
nKV, hd, T = 2, 16, 3
qkv = torch.randn(T, 4 * nKV * hd // 2 + 2 * nKV * hd, device=dev)[:, :(2 + 2 * nKV) * hd].contiguous()
q = torch.empty(T, 2 * hd, device=dev)
kc = torch.zeros(4, nKV, 64, hd, device=dev); vc = torch.zeros_like(kc)
i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)
pages = i32([[1, 9]])                                       # page 9 does not exist (4 pages)
ops.qkv_to_cache(qkv, q, kc, vc, i32([0, 0, 0]), i32([5, 63, 64]), pages, 2, nKV, hd, 1.0)
torch.cuda.synchronize()
st = ops.bounds_status(clear=True)
assert any(v[0] == "page number" and v[1] == 9 and v[2] == 4 for v in st.values()), st
assert kc[1, :, 5].abs().sum() > 0 and kc[1, :, 63].abs().sum() > 0           # the good positions were written
print("ok")
'''


def test_kernels_record_bad_indices_and_never_use_them():
    env = dict(os.environ, GOPHERLLM_DEBUG_BOUNDS="1")
    r = subprocess.run([sys.executable, "-c", SCRIPT, ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout[-2000:] + r.stderr[-4000:]
