"""Weights by tensor name: checking a model folder against what the model's
parts declare, loading, and the seeded random-weights mode.

The reference looks tensors up by name in the file's table (model.go:2260-2266,
2357-2473) and fails on the first problem ("missing tensor: %s",
model.go:2360; "phi2 requires %d-element output.bias", model.go:1903).  Here all
problems of a folder are collected into one error: missing tensors, tensors the
model does not know, and wrong shapes.
"""
from __future__ import annotations

import hashlib
import json
import os
from typing import Callable, Dict, Iterator, List, Optional, Tuple

import torch

from ..parts.base import ParamSpec
from .safetensors_io import TensorEntry, TensorFile, index_folder, write_file

STORAGE_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16,
                  "bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}


class WeightsError(ValueError):
    """A model folder does not hold what the model needs."""

    def __init__(self, folder: str, missing: List[str], unexpected: List[str], wrong: List[str]):
        self.missing, self.unexpected, self.wrong = missing, unexpected, wrong
        lines = [f"{folder}: the weights do not fit the model"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes or types ({len(wrong)}): " + "; ".join(wrong))
        super().__init__("\n".join(lines))


def tensor_table(model_parameters: Dict[str, ParamSpec], names) -> Dict[str, Tuple[str, ParamSpec]]:
    """file tensor name -> (model parameter key, spec).  Keys are "embedding", "positions",
    "final_norm/<p>", "head/<p>" and "layers/<i>/<slot>/<p>", where <p> may itself be a path
    ("sub/weight": a part inside the slot's part); ``names.layer`` gets it with dots for slashes,
    the way a part spells its own nested parameters ("q_norm.weight")."""
    table: Dict[str, Tuple[str, ParamSpec]] = {}
    for key, spec in model_parameters.items():
        parts = key.split("/")
        if parts[0] == "embedding" and len(parts) == 1:
            name = names.embedding
        elif parts[0] == "positions" and len(parts) == 1:
            name = getattr(names, "positions", None)
            if name is None:
                raise KeyError("the model has a position table but its tensor names give no `positions`")
        elif parts[0] == "final_norm" and len(parts) >= 2:
            name = f"{names.final_norm}.{'.'.join(parts[1:])}"
        elif parts[0] == "head" and len(parts) >= 2:
            name = f"{names.head}.{'.'.join(parts[1:])}"
        elif parts[0] == "layers" and len(parts) >= 4:
            name = names.layer(int(parts[1]), parts[2], ".".join(parts[3:]))
        else:
            raise KeyError(f"model parameter {key!r} has no tensor name")
        if name in table:
            raise KeyError(f"tensor name {name} is used by two parameters")
        table[name] = (key, spec)
    return table


_WIDE = (torch.float32, torch.float64)
_HALF = (torch.bfloat16, torch.float16)


def resident_dtype(spec: ParamSpec, stored: torch.dtype, compute: torch.dtype,
                   declared: Optional[torch.dtype] = None, keep_stored: Optional[bool] = None) -> torch.dtype:
    """The type a tensor is held in.  Integer tables: int32.  1-D tensors: float32
    (model.go:2519-2528).  Matrices: float32 in the 32-bit path.  In the bfloat16 path every stored
    type is brought to the compute type when loading, as the reference expands F32, F16, BF16 and F64
    alike to its compute type (model.go:2399-2436): a matrix stored as float16 (the published Phi
    checkpoints) is rounded to bfloat16, nearest even, and so is a checkpoint that is 32-bit as a whole
    (``declared``, the folder's torch_dtype, is 32-bit or unknown).  One exception: a matrix stored in
    32-bit inside a checkpoint that declares a 16-bit type was stored wider on purpose and stays
    float32 (its products then run on the 32-bit CUDA-core kernel).  ``keep_stored`` True keeps every
    matrix that is not stored as bfloat16 in float32 instead; False rounds all of them."""
    if spec.kind == "table_int":
        return torch.int32
    if spec.kind == "vector" or compute == torch.float32:
        return torch.float32
    if stored == torch.bfloat16:
        return torch.bfloat16
    if keep_stored is None:
        keep_stored = stored in _WIDE and declared in _HALF
    return torch.float32 if keep_stored else torch.bfloat16


def split_fused(entries: Dict[str, TensorEntry], table: Dict[str, Tuple[str, ParamSpec]],
                fused: Optional[Dict[str, List[str]]], wrong: List[str]) -> Dict[str, TensorEntry]:
    """A file may hold several declared tensors as one, their rows one after the other (the reference
    takes a fused attn_qkv or split attn_q/k/v, whichever the file has, model.go:2046-2065, and cuts a
    fused bias by row ranges, model.go:2222-2227).  ``fused``: file tensor name -> names of the declared
    tensors it holds, in row order.  Where the fused tensor is present and none of its parts is, the
    parts become entries of their own that point into its bytes (rows are contiguous in the file)."""
    if not fused:
        return entries
    entries = dict(entries)
    for fname, parts in fused.items():
        e = entries.get(fname)
        if e is None or any(p in entries for p in parts) or any(p not in table for p in parts):
            continue
        shapes = [tuple(table[p][1].shape) for p in parts]
        rows = sum(s[0] for s in shapes)
        if any(s[1:] != e.shape[1:] for s in shapes) or e.shape[0] != rows:
            wrong.append(f"{fname} is {list(e.shape)}, the model wants {[rows, *shapes[0][1:]]} "
                         f"(the rows of {', '.join(parts)})")
            del entries[fname]
            for p, s in zip(parts, shapes):               # reported once, as the fused tensor
                entries[p] = TensorEntry(p, e.dtype, s, e.begin, e.begin, e.file)
            continue
        row_bytes = (e.end - e.begin) // max(1, e.shape[0])
        at = e.begin
        for p, s in zip(parts, shapes):
            entries[p] = TensorEntry(p, e.dtype, s, at, at + s[0] * row_bytes, e.file)
            at += s[0] * row_bytes
        del entries[fname]
    return entries


def check_folder(folder: str, table: Dict[str, Tuple[str, ParamSpec]], ignore: Tuple[str, ...] = (),
                 fused: Optional[Dict[str, List[str]]] = None):
    """Compare the folder's tensor table with what the model declares."""
    wrong: List[str] = []
    entries = split_fused(index_folder(folder), table, fused, wrong)
    missing = sorted(n for n, (_, spec) in table.items() if n not in entries and not spec.optional)
    unexpected = sorted(n for n in entries if n not in table and n not in ignore)
    for n, (_, spec) in sorted(table.items()):
        e = entries.get(n)
        if e is None:
            continue
        if tuple(e.shape) != tuple(spec.shape):
            wrong.append(f"{n} is {list(e.shape)}, the model wants {list(spec.shape)}")
        elif spec.kind != "table_int" and e.dtype not in ("F32", "F16", "BF16", "F64"):
            wrong.append(f"{n} is stored as {e.dtype}, not a floating-point type")
    if missing or unexpected or wrong:
        raise WeightsError(folder, missing, unexpected, wrong)
    return entries


def load_folder(folder: str, table: Dict[str, Tuple[str, ParamSpec]], compute: torch.dtype, device,
                ignore: Tuple[str, ...] = (), progress: Optional[Callable[[str], None]] = None,
                fused: Optional[Dict[str, List[str]]] = None, declared: Optional[torch.dtype] = None,
                keep_stored: Optional[bool] = None) -> Tuple[Dict[str, torch.Tensor], int]:
    """Tensors by model parameter key, on ``device``, in their resident types (``resident_dtype``);
    and the bytes read.  Tensors are copied as stored and rounded on the device."""
    entries = check_folder(folder, table, ignore, fused)
    out: Dict[str, torch.Tensor] = {}
    nbytes = 0
    rounded: Dict[str, int] = {}
    with TensorFile(entries) as tf:
        for i, (name, (key, spec)) in enumerate(sorted(table.items())):
            if name not in entries:          # optional and absent
                out[key] = torch.zeros(spec.shape, dtype=resident_dtype(spec, torch.float32, compute), device=device)
                continue
            t = tf.get(name)
            nbytes += t.numel() * t.element_size()
            want = resident_dtype(spec, t.dtype, compute, declared, keep_stored)
            if spec.kind == "matrix" and want == torch.bfloat16 and t.dtype != torch.bfloat16:
                label = str(t.dtype).replace("torch.", "")
                rounded[label] = rounded.get(label, 0) + 1
            out[key] = t.to(device=device).to(dtype=want).contiguous()
            if progress and i % 64 == 0:
                progress(f"loaded {i + 1}/{len(table)} tensors")
    if progress and rounded:
        progress("rounded to bfloat16 (nearest even) at load: "
                 + ", ".join(f"{n} matrices stored as {k}" for k, n in sorted(rounded.items())))
    return out, nbytes


# ---------------------------------------------------------------------------
# random weights
# ---------------------------------------------------------------------------
def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{int(seed)}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def random_tensor(name: str, spec: ParamSpec, seed: int, sigma: float, storage: torch.dtype) -> torch.Tensor:
    """One declared tensor of the random-weights mode, drawn on the CPU from a generator seeded by
    (seed, name), in float32, and rounded to ``storage``."""
    if spec.kind == "table_int":
        return torch.zeros(spec.shape, dtype=torch.int32)
    g = torch.Generator(device="cpu")
    g.manual_seed(_tensor_seed(seed, name))
    z = torch.randn(spec.shape, generator=g, dtype=torch.float32)
    if spec.init == "normal":
        t = z.mul_(sigma)
    elif spec.init in ("bias", "beta"):
        t = z.mul_(0.02)
    elif spec.init == "gamma":
        t = z.mul_(0.02).add_(1.0)
    elif spec.init == "zeros":
        t = z.zero_()
    else:
        raise ValueError(f"{name}: unknown initialisation {spec.init!r}")
    return t.to(storage)


def random_tensors(table: Dict[str, Tuple[str, ParamSpec]], seed: int, sigma: float,
                   storage: torch.dtype, workers: int = 0) -> Iterator[Tuple[str, torch.Tensor]]:
    """(name, tensor) for every declared tensor, in name order, each from a CPU generator seeded by
    (seed, name): values depend neither on the order of generation nor on who asks, so a folder
    written with a seed and a model built in memory with it hold the same tensors.  Matrices
    N(0, sigma); biases and norm offsets N(0, 0.02); norm scales 1 + N(0, 0.02).  ``workers`` > 1
    draws that many tensors at a time on threads (drawing is the slow part of a large model)."""
    items = sorted(table.items())
    if workers <= 1 or len(items) < 2:
        for name, (_, spec) in items:
            yield name, random_tensor(name, spec, seed, sigma, storage)
        return
    from concurrent.futures import ThreadPoolExecutor
    ahead = 2 * workers                       # tensors drawn but not yet taken: bounds the host memory held
    with ThreadPoolExecutor(max_workers=workers) as pool:
        pending = []
        it = iter(items)

        def submit():
            nxt = next(it, None)
            if nxt is not None:
                name, (_, spec) = nxt
                pending.append((name, pool.submit(random_tensor, name, spec, seed, sigma, storage)))

        for _ in range(ahead):
            submit()
        while pending:
            name, fut = pending.pop(0)
            submit()
            yield name, fut.result()


def write_model_folder(folder: str, config_dict: dict, table: Dict[str, Tuple[str, ParamSpec]],
                       seed: int, sigma: float, storage: torch.dtype, workers: int = 0) -> None:
    """config.json and model.safetensors of a random model."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=2, sort_keys=True)
    write_file(os.path.join(folder, "model.safetensors"),
               random_tensors(table, seed, sigma, storage, workers),
               metadata={"format": "pt", "seed": seed})
