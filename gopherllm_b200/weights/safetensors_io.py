"""Reading and writing the safetensors container.

Layout of a file: 8 bytes little-endian header length n, n bytes of JSON
``{name: {"dtype", "shape", "data_offsets": [begin, end]}, "__metadata__": …}``,
then the tensors' raw little-endian bytes; offsets count from the end of the
header.  The reference's container is GGUF (gguf.go:496-569: header, key/value
metadata, tensor table, aligned data); the checks it makes on every tensor
(offset in range, data inside the file: model.go:2376-2387) are made here too.
"""
from __future__ import annotations

import json
import mmap
import os
import struct
from dataclasses import dataclass
from typing import Dict, Iterable, List, Tuple

import numpy as np
import torch

_DTYPES = {
    "F64": (torch.float64, 8), "F32": (torch.float32, 4), "F16": (torch.float16, 2),
    "BF16": (torch.bfloat16, 2), "I64": (torch.int64, 8), "I32": (torch.int32, 4),
    "I16": (torch.int16, 2), "I8": (torch.int8, 1), "U8": (torch.uint8, 1),
    "BOOL": (torch.bool, 1),
}
_NAMES = {v[0]: k for k, v in _DTYPES.items()}


@dataclass(frozen=True)
class TensorEntry:
    name: str
    dtype: str                 # safetensors dtype code, e.g. "BF16"
    shape: Tuple[int, ...]
    begin: int                 # byte offsets inside the file
    end: int
    file: str

    @property
    def torch_dtype(self) -> torch.dtype:
        return _DTYPES[self.dtype][0]

    @property
    def numel(self) -> int:
        n = 1
        for s in self.shape:
            n *= s
        return n


def read_header(path: str) -> Tuple[Dict[str, TensorEntry], dict]:
    """Tensor table and metadata of one file, without touching tensor data."""
    size = os.path.getsize(path)
    with open(path, "rb") as f:
        head = f.read(8)
        if len(head) < 8:
            raise ValueError(f"{path}: too short for a safetensors header")
        (n,) = struct.unpack("<Q", head)
        if n > size - 8 or n > (1 << 30):
            raise ValueError(f"{path}: header length {n} exceeds file length {size}")
        try:
            table = json.loads(f.read(n).decode("utf-8"))
        except (UnicodeDecodeError, json.JSONDecodeError) as e:
            raise ValueError(f"{path}: header is not JSON: {e}") from None
    base = 8 + n
    meta = table.pop("__metadata__", {}) or {}
    entries: Dict[str, TensorEntry] = {}
    for name, info in table.items():
        dt = info.get("dtype")
        if dt not in _DTYPES:
            raise ValueError(f"unsupported tensor type for {name}: {dt}")
        shape = tuple(int(s) for s in info["shape"])
        b, e = (int(x) for x in info["data_offsets"])
        ent = TensorEntry(name, dt, shape, base + b, base + e, path)
        if b < 0 or e < b:
            raise ValueError(f"tensor {name} offset out of range")
        if base + e > size:
            raise ValueError(f"tensor {name} exceeds file length")
        if ent.numel * _DTYPES[dt][1] != e - b:
            raise ValueError(f"tensor {name}: {e - b} bytes do not hold shape {list(shape)} of {dt}")
        entries[name] = ent
    return entries, meta


def index_folder(folder: str) -> Dict[str, TensorEntry]:
    """Tensor table of a model folder: ``model.safetensors``, or the shards
    that ``model.safetensors.index.json`` lists."""
    single = os.path.join(folder, "model.safetensors")
    index = os.path.join(folder, "model.safetensors.index.json")
    files: List[str]
    if os.path.isfile(single):
        files = [single]
    elif os.path.isfile(index):
        with open(index, "r", encoding="utf-8") as f:
            wm = json.load(f).get("weight_map", {})
        files = sorted({os.path.join(folder, v) for v in wm.values()})
    else:
        raise FileNotFoundError(f"{folder}: no model.safetensors")
    entries: Dict[str, TensorEntry] = {}
    for path in files:
        part, _ = read_header(path)
        for k, v in part.items():
            if k in entries:
                raise ValueError(f"tensor {k} appears in two files")
            entries[k] = v
    return entries


class TensorFile:
    """Memory-mapped view of the files of a folder; ``get`` returns a CPU tensor
    that aliases the mapping (copy it, or move it to a device, before close)."""

    def __init__(self, entries: Dict[str, TensorEntry]):
        self.entries = entries
        self._maps: Dict[str, Tuple[object, mmap.mmap]] = {}

    def _map(self, path: str) -> mmap.mmap:
        if path not in self._maps:
            f = open(path, "rb")
            self._maps[path] = (f, mmap.mmap(f.fileno(), 0, access=mmap.ACCESS_READ))
        return self._maps[path][1]

    def get(self, name: str) -> torch.Tensor:
        e = self.entries[name]
        if e.numel == 0:
            return torch.empty(e.shape, dtype=e.torch_dtype)
        buf = np.frombuffer(self._map(e.file), dtype=np.uint8, count=e.end - e.begin, offset=e.begin)
        # torch has no view of read-only memory; the copy is the load itself
        t = torch.from_numpy(buf.copy())
        return t.view(e.torch_dtype).reshape(e.shape)

    def close(self) -> None:
        for f, m in self._maps.values():
            m.close()
            f.close()
        self._maps.clear()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_file(path: str, tensors: Iterable[Tuple[str, torch.Tensor]], metadata: dict = None) -> None:
    """Write tensors (name, CPU tensor) to one safetensors file.  Tensors are
    taken one at a time so a generator can stream a large model."""
    tmp = path + ".tmp"
    table = {}
    offset = 0
    body = tmp + ".body"
    with open(body, "wb") as f:
        for name, t in tensors:
            t = t.detach().contiguous().cpu()
            if t.dtype not in _NAMES:
                raise ValueError(f"tensor {name}: dtype {t.dtype} cannot be stored")
            raw = t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""
            f.write(raw)
            table[name] = {"dtype": _NAMES[t.dtype], "shape": list(t.shape),
                           "data_offsets": [offset, offset + len(raw)]}
            offset += len(raw)
    if metadata:
        table["__metadata__"] = {str(k): str(v) for k, v in metadata.items()}
    head = json.dumps(table, separators=(",", ":")).encode("utf-8")
    head += b" " * ((8 - len(head) % 8) % 8)
    with open(tmp, "wb") as out:
        out.write(struct.pack("<Q", len(head)))
        out.write(head)
        with open(body, "rb") as f:
            while True:
                chunk = f.read(1 << 24)
                if not chunk:
                    break
                out.write(chunk)
    os.remove(body)
    os.replace(tmp, path)
