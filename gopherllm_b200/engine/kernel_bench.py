"""Isolated timing of one layer's products, in the manner of the reference's
--kernel-bench (kernel_bench.go:28-183: embedding row, the matvecs of one layer,
the output projection; "llm-kernel-bench.v1" JSON).  Here each row is the kernel
the engine would launch for a decode step of ``batch`` tokens, timed with CUDA
events, with the bytes it streams and the bandwidth that makes."""
from __future__ import annotations

import json
from typing import List

import torch

from .. import ops


def _time(fn, runs: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(runs):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def kernel_bench_rows(model, runs: int, layer: int, batch: int = 1) -> List[dict]:
    eng = model.engine
    net = eng.model
    dt, dev = eng.act_dtype, eng.device
    rows = []

    def row(name, weight, fn):
        total = _time(fn, runs)
        nbytes = weight.numel() * weight.element_size()
        rows.append({"name": name, "dtype": str(weight.dtype).replace("torch.", ""), "rows": weight.shape[0],
                     "cols": weight.shape[1], "runs": runs, "avg_ms": total / runs, "total_ms": total,
                     "gb_per_s": nbytes / (total / runs / 1e3) / 1e9})

    toks = torch.zeros(batch, dtype=torch.int32, device=dev)
    row("token_embd.row", net.embedding, lambda: ops.embed(net.embedding, toks))
    if net.blocks:
        blk = net.blocks[max(0, min(layer, len(net.blocks) - 1))]

        def x(n):
            return (torch.arange(batch * n, device=dev, dtype=torch.float32).reshape(batch, n) % 17 - 8).mul(0.01).to(dt)

        # every product the layer's parts declare, whatever kinds they are: each as the kernel a step
        # of ``batch`` tokens would launch for it
        for name, w, b, act in blk.products():
            xin = x(w.shape[1])
            # a product as wide as the model adds onto the 32-bit residual stream; others feed the next product
            out_dt = torch.float32 if w.shape[0] == net.spec.hidden else dt
            row(name.replace(".", "_"), w, lambda xin=xin, w=w, b=b, act=act, out_dt=out_dt: ops.linear(xin, w, b, act=act, out_dtype=out_dt))
    xh = (torch.ones(batch, net.head_weight.shape[1], device=dev) * 0.01).to(dt)
    row("output", net.head_weight, lambda: ops.linear(xh, net.head_weight, net.head_bias, out_dtype=torch.float32))
    return rows


def run_kernel_bench(model, path: str, runs: int, layer: int, as_json: bool, batch: int = 1) -> int:
    if runs <= 0:
        raise SystemExit("--kernel-bench-runs must be greater than 0")
    rows = kernel_bench_rows(model, runs, layer, batch)
    spec = model.spec
    if as_json:
        print(json.dumps({"type": "gopherllm.kernel_benchmark", "format": "llm-kernel-bench.v1",
                          "runtime": "gopherllm_b200",
                          "model": {"path": path, "arch": model.architecture.name, "dim": spec.hidden,
                                    "layers": len(spec.layers), "dtype": model.info.dtype},
                          "layer": layer, "runs": runs, "batch": batch, "kernels": rows}, indent=2))
        return 0
    print(f"Kernel benchmark format=llm-kernel-bench.v1 runtime=gopherllm_b200 layer={layer} runs={runs}")
    for r in rows:
        print(f"{r['name']} dtype={r['dtype']} rows={r['rows']} cols={r['cols']} avg={r['avg_ms']:.3f}ms "
              f"total={r['total_ms']:.3f}ms {r['gb_per_s']:.0f}GB/s")
    return 0
