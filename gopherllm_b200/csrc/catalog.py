"""Which libraries exist: (source file, preprocessor definitions) pairs."""
from __future__ import annotations

from typing import Iterable, Iterator, Tuple

# libraries that do not depend on a model's sizes
GENERAL = ("rowwise.cu", "qkv_cache.cu", "attention_generic.cu", "gemm_simt.cu", "gemm_skinny.cu", "gemm_stream.cu",
           "gemm_tcgen05.cu", "sampling.cu")

# libraries compiled once per head size (GL_HEAD_DIM)
PER_HEAD_DIM: Tuple[str, ...] = ("attention_decode.cu", "attention_prefill.cu", "attention_prefill_tc.cu",
                                  "decode_layer.cu")
# libraries that take only some head sizes
MAX_HEAD_DIM = {"attention_prefill_tc.cu": 128, "decode_layer.cu": 128}


def head_dim_defines(head_dim: int) -> Tuple[str, ...]:
    return (f"GL_HEAD_DIM={int(head_dim)}",)


def all_libraries(head_dims: Iterable[int] = ()) -> Iterator[Tuple[str, Tuple[str, ...]]]:
    for src in GENERAL:
        yield src, ()
    for hd in sorted(set(int(h) for h in head_dims)):
        for src in PER_HEAD_DIM:
            if hd <= MAX_HEAD_DIM.get(src, 1 << 30):
                yield src, head_dim_defines(hd)
