"""Writes tests/golden/plain_tiny.json: a few logits of the plain implementation
(tests/plain_phi.py) on the tiny configurations with their seeded random weights.

The reference (SimonWaldherr/GopherLLM) is Go and no Go toolchain exists on the
machines this was made on, so these numbers do not come from a run of its code: they
pin the plain implementation and the random-weights mode against accidental change.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))


def compute():
    import plain_phi
    import tiny
    out = {}
    for name in ("A", "B", "C"):
        cfg, W = plain_phi.read_folder(tiny.folder(name))
        toks = tiny.prompt(np.random.default_rng(100), 24, cfg["vocab_size"])
        logits = plain_phi.phi_logits(toks, W, cfg).numpy()
        out[name] = {"tokens": toks, "argmax": [int(i) for i in logits.argmax(-1)],
                     "last_row_first_8": [float(f"{v:.6f}") for v in logits[-1, :8]],
                     "row_sums": [float(f"{v:.5f}") for v in logits.sum(-1)]}
    return out


if __name__ == "__main__":
    with open(os.path.join(HERE, "plain_tiny.json"), "w") as f:
        json.dump(compute(), f, indent=1)
    print("wrote plain_tiny.json")
