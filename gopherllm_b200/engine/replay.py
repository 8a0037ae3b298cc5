"""Trace replay: feed given token ids through a model step by step and write logits.

Nothing is sampled.  The program drives the library's own loader, cache, step
function and kernels; it has none of its own.  Steps arrive on standard input,
one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step in which logits are wanted, ``<out>/<step>.f32`` receives them as
little-endian float32 [wanted, vocab], in the order of the entries and of
``want``.  After every step a line ``done <step>`` is printed and flushed.
The reference's closest relative is its parity helper, which feeds the same
tokens one by one and as a batch and compares logits and cache
(arch_improvements_test.go:129-164).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict

import numpy as np


def run(model, lines, out_dir: str, emit=print) -> None:
    """Replay ``lines`` (an iterable of JSON strings) on a loaded Model."""
    os.makedirs(out_dir, exist_ok=True)
    slots: Dict[str, int] = {}
    check = getattr(getattr(model, "engine", None), "check_device", lambda: None)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        runs, want = [], []
        for e in rec.get("entries", []):
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = model.open_sequence()
            runs.append((slots[rid], [int(t) for t in e["tokens"]]))
            want.append([int(i) for i in e.get("want", [])])
        if runs:
            logits = model.step(runs, want)
            if logits.shape[0] > 0:
                arr = logits.detach().float().cpu().numpy().astype("<f4", copy=False)
                check()                          # the copy waited for the step: a kernel that gave up is an error
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid in slots:
                model.close_sequence(slots.pop(rid))
        emit(f"done {step}")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to 64")
    ap.add_argument("--device", default="cuda:0")
    args = ap.parse_args(argv)

    def log(msg):
        print(f"[trace_run] {msg}", file=sys.stderr, flush=True)

    from ..api import load
    model = load(args.model, dtype=args.dtype, max_tokens=args.max_tokens, device=args.device, log=log)

    def emit(s):
        sys.stdout.write(s + "\n")
        sys.stdout.flush()

    run(model, sys.stdin, args.out, emit)
    return 0


if __name__ == "__main__":
    sys.exit(main())
