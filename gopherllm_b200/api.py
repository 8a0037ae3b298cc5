"""The Python entry point: open a model folder, step it, generate with it.

It mirrors the reference's package API (api.go): ``load`` is ``Open``
(api.go:105-115), ``Model.generate`` is ``Model.Generate`` (api.go:257-259) with
the same option names in snake case (WithMaxTokens … WithSeed, api.go:182-221),
``Model.info`` is ``Info`` (api.go:165), ``Model.close`` is ``Close``
(api.go:156).  Prompts are token ids: tokenizers are outside this library.
"""
from __future__ import annotations

import os
import time
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence

import torch

from .cache.sequence_cache import SequenceCache
from .config import load_config, read_config_json
from .config.registry import Architecture
from .engine.model import DecoderModel
from .engine.step import Engine
from .weights.loader import STORAGE_DTYPES, load_folder, tensor_table, write_model_folder

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
           "float32": torch.float32, "fp32": torch.float32, "f32": torch.float32}


@dataclass
class LoadInfo:
    """What loading cost (the reference's LoadInfo, api.go:25-28, runtime.go:658-705)."""
    path: str
    architecture: str
    dtype: str
    load_seconds: float
    file_bytes: int
    weight_bytes: int
    cache_bytes: int
    max_tokens: int


def _require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("gopherllm_b200 runs on a CUDA device only (there is no CPU path)")
    if not torch.cuda.is_available():
        raise RuntimeError("no CUDA device is available: gopherllm_b200 needs a B200 (sm_100a)")
    return device


def compute_dtype(dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype in (torch.bfloat16, torch.float32):
            return dtype
    elif str(dtype).lower() in _DTYPES:
        return _DTYPES[str(dtype).lower()]
    raise ValueError(f"dtype {dtype!r}: choose bfloat16 or float32")


class Model:
    """A loaded model with its cache.  Not thread-safe: one step at a time."""

    def __init__(self, arch: Architecture, config, engine: Engine, info: LoadInfo):
        self.architecture, self.config, self.engine, self.info = arch, config, engine, info
        self.spec = engine.model.spec
        self._closed = False

    # sequences and steps ------------------------------------------------
    def open_sequence(self) -> int:
        return self.engine.open()

    def close_sequence(self, slot: int) -> None:
        self.engine.close(slot)

    def step(self, runs, want=None) -> torch.Tensor:
        """See Engine.step."""
        return self.engine.step(runs, want)

    def generate(self, prompts, **options):
        """Generate for one prompt (a list of token ids) or several (a list of
        lists).  Options: max_tokens, temperature, top_p, top_k, min_p,
        repeat_penalty, seed, stop_tokens, should_stop, on_token (called with
        (request index, token) for every token as it is emitted; returning
        False cancels).  Returns a GenerationResult, or a list of them."""
        from .engine.generate import GenerationOptions, generate
        single = len(prompts) > 0 and not isinstance(prompts[0], (list, tuple))
        opts = options.pop("options", None) or GenerationOptions.from_kwargs(self.spec, **options)
        results = generate(self.engine, [list(prompts)] if single else [list(p) for p in prompts], opts)
        return results[0] if single else results

    def close(self) -> None:
        """Release the weights and the cache."""
        if not self._closed:
            self.engine.model = None
            self.engine.cache = None
            self._closed = True
            torch.cuda.empty_cache()


def build_model(arch: Architecture, config) -> DecoderModel:
    return DecoderModel(arch.build_spec(config))


def load(path: str, dtype="bfloat16", max_tokens: Optional[int] = None, device="cuda:0",
         max_slots: Optional[int] = None, log: Optional[Callable[[str], None]] = None,
         keep_stored: Optional[bool] = None) -> Model:
    """Open a model folder (config.json + model.safetensors).

    dtype: "bfloat16" (the serving kernels) or "float32" (everything in true
    32-bit).  max_tokens: positions the cache holds for all live sequences
    together, each rounded up to 64 (default: 8 sequences of the model's full
    length).  Silent unless ``log`` is given (the reference: api.go:44-54).
    With dtype "bfloat16", matrices stored in another type (float16 as in the
    published Phi checkpoints, or a checkpoint that is 32-bit as a whole) are rounded
    to bfloat16 when loading, and ``log`` is told so; a matrix stored in 32-bit
    inside a 16-bit checkpoint stays 32-bit.  keep_stored=True keeps every matrix
    that is not stored as bfloat16 in 32-bit (exact, and slow: such products run on
    CUDA cores); keep_stored=False rounds every matrix.
    """
    device = _require_cuda(device)
    cdt = compute_dtype(dtype)
    t0 = time.time()
    arch, config = load_config(path)
    model = build_model(arch, config)
    names = arch.tensor_names(config)
    table = tensor_table(model.parameters(), names)
    ignore = ("lm_head.weight",) if model.spec.tie_embeddings else ()
    fused = names.fused() if hasattr(names, "fused") else None
    with torch.cuda.device(device):
        raw = read_config_json(path)       # the type the checkpoint declares, None if it declares none
        declared = STORAGE_DTYPES.get(str(raw.get("torch_dtype", raw.get("dtype"))))
        tensors, nbytes = load_folder(path, table, cdt, device, ignore=ignore, progress=log, fused=fused,
                                      declared=declared, keep_stored=keep_stored)
        model.load(tensors)
        del tensors
        if max_tokens is None:
            max_tokens = 8 * model.spec.max_positions
        cache = SequenceCache(model.cache_requests(), max_tokens, model.spec.max_positions,
                              cdt, device, max_slots=max_slots)
        engine = Engine(model, cache, cdt, device)
    info = LoadInfo(path=os.path.abspath(path), architecture=arch.name,
                    dtype="bfloat16" if cdt == torch.bfloat16 else "float32",
                    load_seconds=time.time() - t0, file_bytes=nbytes,
                    weight_bytes=model.weight_bytes(), cache_bytes=cache.bytes(), max_tokens=max_tokens)
    if log:
        log(f"loaded {arch.name} from {path} in {info.load_seconds:.2f} s "
            f"({info.weight_bytes / 1e9:.2f} GB weights, {info.cache_bytes / 1e9:.2f} GB cache)")
    return Model(arch, config, engine, info)


def _draw_workers() -> int:
    return max(1, min(16, (os.cpu_count() or 1)))


def load_random(config, seed: int = 0, dtype="bfloat16", max_tokens: Optional[int] = None,
                device="cuda:0", max_slots: Optional[int] = None, layers: Optional[int] = None) -> Model:
    """A model with seeded random weights built in memory: tensor for tensor what
    ``write_random_model(folder, config, seed)`` writes and ``load(folder, dtype)`` then holds (the
    tensors are drawn on the CPU from the same per-tensor generators, several at a time, and rounded
    by the same rule), without the folder.  ``layers`` keeps only the first so many layers (for
    machines or tests short of memory): those layers, the embedding and the head are the same
    tensors as in the full model, since each is drawn from (seed, its own name)."""
    from .config.registry import architecture_from_config
    from .weights.loader import random_tensors, resident_dtype
    device = _require_cuda(device)
    cdt = compute_dtype(dtype)
    t0 = time.time()
    raw = dict(config if isinstance(config, dict) else config.to_dict())
    if layers is not None:
        raw["num_hidden_layers"] = int(layers)
    arch = architecture_from_config(raw)
    cfg = arch.config_class.from_dict(raw)
    model = build_model(arch, cfg)
    table = tensor_table(model.parameters(), arch.tensor_names(cfg))
    storage = STORAGE_DTYPES.get(str(getattr(cfg, "torch_dtype", "bfloat16")), torch.bfloat16)
    sigma = float(getattr(cfg, "initializer_range", 0.02))
    tensors = {}
    with torch.cuda.device(device):
        for name, t in random_tensors(table, seed, sigma, storage, workers=_draw_workers()):
            key, spec = table[name]
            tensors[key] = t.to(device).to(resident_dtype(spec, storage, cdt, storage)).contiguous()
        model.load(tensors)
        del tensors
        if max_tokens is None:
            max_tokens = 8 * model.spec.max_positions
        cache = SequenceCache(model.cache_requests(), max_tokens, model.spec.max_positions,
                              cdt, device, max_slots=max_slots)
        engine = Engine(model, cache, cdt, device)
    info = LoadInfo(path=f"random:{seed}", architecture=arch.name,
                    dtype="bfloat16" if cdt == torch.bfloat16 else "float32",
                    load_seconds=time.time() - t0, file_bytes=0, weight_bytes=model.weight_bytes(),
                    cache_bytes=cache.bytes(), max_tokens=max_tokens)
    return Model(arch, cfg, engine, info)


def write_random_model(folder: str, config, seed: int = 0) -> None:
    """Write config.json and model.safetensors of a model with seeded random
    weights.  ``config`` is a config.json dict or a typed configuration.  Matrices
    are N(0, initializer_range), stored in the config's torch_dtype."""
    from .config.registry import architecture_from_config
    raw = config if isinstance(config, dict) else config.to_dict()
    arch = architecture_from_config(raw)
    cfg = arch.config_class.from_dict(raw)
    model = build_model(arch, cfg)
    table = tensor_table(model.parameters(), arch.tensor_names(cfg))
    storage = STORAGE_DTYPES.get(str(getattr(cfg, "torch_dtype", "bfloat16")), torch.bfloat16)
    write_model_folder(folder, cfg.to_dict(), table, seed, float(getattr(cfg, "initializer_range", 0.02)),
                       storage, workers=_draw_workers())
