"""Python face of the CUDA kernels.

Every function checks sizes, element types and devices on the host, then calls
one launcher on the current CUDA stream.  There is no CPU implementation and no
library fallback: a tensor that is not on a CUDA device, or a library that does
not build, is an error.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, byref, c_float, c_int, c_void_p
from typing import Optional

import torch

from .csrc import build, catalog

PAGE = 64                      # tokens per cache page (GL_PAGE)
F32, BF16 = 0, 1
ACTIVATIONS = {"none": 0, None: 0, "gelu_new": 1, "gelu_pytorch_tanh": 1, "gelu": 2, "relu": 3}
SAMPLE_WINDOW = 64             # tokens the repeat penalty looks back on (runtime.go:27)
SAMPLE_KMAX = 1024

_ERRORS = {
    -1: "this combination of element types is not built",
    -2: "a size the kernel does not take",
    -3: "a pointer or stride is not aligned as the kernel requires",
    -4: "the launch failed (cudaGetLastError)",
    -5: "the kernel needs more shared memory than the device allows",
    -6: "a CUDA driver entry point is missing or failed",
    -7: "the call needs more scratch than the library's built-in array holds",
}


class KernelError(RuntimeError):
    pass


LAUNCHES = 0       # kernels launched through this module since it was last set to 0


def _check(code: int, what: str, kernels: int = 1) -> None:
    global LAUNCHES
    LAUNCHES += kernels
    if _TAPE is not None and _TAPE.calls and _TAPE.calls[-1][2] is None:
        _TAPE.calls[-1][2:] = [what, kernels]
    if code != 0:
        raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")


# ---------------------------------------------------------------------------
# A tape of launches.  The layers of a model are mostly the same block with other tensors; what the
# host does for one of them (checks, sizes, argument records: some 100 us for a block of five kernels,
# more than the kernels take for a short prompt) is the same for the next but for a handful of
# pointers.  So the launches of one block's run can be recorded and repeated for another block of the
# same shape with that block's tensors in place of the first one's.
class _StreamArg(c_void_p):
    """The stream argument of a launch (a repeated launch takes the stream that is current then)."""


class LaunchTape:
    """The launches between ``start()`` and ``stop()``: [function, arguments, name, kernels] each, and
    the tensors that were allocated for them meanwhile (kept alive: a repeat uses them again)."""

    def __init__(self):
        self.calls: list = []
        self.temps: list = []
        self.slots: list = []
        self.streams: list = []

    def start(self) -> "LaunchTape":
        global _TAPE
        if _TAPE is not None:
            raise KernelError("a tape of launches is already being recorded")
        _TAPE = self
        return self

    def stop(self) -> "LaunchTape":
        global _TAPE
        _TAPE = None
        return self

    def _pointers(self):
        """Every place a pointer stands: (holder, attribute), a c_void_p argument or a record's field."""
        for call in self.calls:
            for a in call[1]:
                if isinstance(a, _StreamArg):
                    continue
                if isinstance(a, c_void_p):
                    yield a, "value"
                else:
                    st = getattr(a, "_obj", None)
                    if isinstance(st, Structure):
                        for name, typ in st._fields_:
                            if typ is c_void_p:
                                yield st, name

    def bind(self, ptrs: dict) -> None:
        """``ptrs``: name -> address of the recorded block's tensors.  Finds the places that hold one."""
        by_ptr: dict = {}
        for k, v in ptrs.items():
            if v:
                by_ptr.setdefault(v, k)
        self.slots = [(h, attr, by_ptr[getattr(h, attr)]) for h, attr in self._pointers()
                      if getattr(h, attr) in by_ptr]
        self.streams = [a for call in self.calls for a in call[1] if isinstance(a, _StreamArg)]

    def same_as(self, other: "LaunchTape", mine: dict, theirs: dict) -> bool:
        """Whether ``other``, the tape of another block's own run, is this tape with that block's tensors
        (``theirs``) in place of this one's (``mine``) and its temporaries in place of this one's, and
        nothing else different: then repeating this tape with a third block's tensors is that block's run."""
        if mine.keys() != theirs.keys() or len(self.calls) != len(other.calls) or len(self.temps) != len(other.temps):
            return False
        to: dict = {}
        for k, v in mine.items():
            if bool(v) != bool(theirs[k]) or (v and to.setdefault(v, theirs[k]) != theirs[k]):
                return False
        for a, b in zip(self.temps, other.temps):
            if a.shape != b.shape or a.dtype != b.dtype:
                return False
            to[a.data_ptr()] = b.data_ptr()

        def same_pointer(u, v):
            return (not u and not v) or (bool(u) and to.get(u, u) == v)

        for (f0, a0, w0, k0), (f1, a1, w1, k1) in zip(self.calls, other.calls):
            if f0 is not f1:
                return False
            if w0 != w1 or k0 != k1 or len(a0) != len(a1):
                return False
            for u, v in zip(a0, a1):
                if type(u) is not type(v):
                    return False
                if isinstance(u, _StreamArg):
                    continue
                if isinstance(u, c_void_p):
                    if not same_pointer(u.value, v.value):
                        return False
                    continue
                su, sv = getattr(u, "_obj", None), getattr(v, "_obj", None)
                if isinstance(su, Structure):
                    if type(su) is not type(sv):
                        return False
                    for name, typ in su._fields_:
                        x, y = getattr(su, name), getattr(sv, name)
                        if typ is c_void_p:
                            if not same_pointer(x, y):
                                return False
                        elif hasattr(x, "__len__"):
                            if list(x) != list(y):
                                return False
                        elif x != y:
                            return False
                elif getattr(u, "value", u) != getattr(v, "value", v):
                    return False
        return True

    def repeat(self, ptrs: dict) -> None:
        """Launch everything again with these tensors in the recorded block's places."""
        global TAPE_REPEATS
        TAPE_REPEATS += 1
        for h, attr, key in self.slots:
            setattr(h, attr, ptrs[key] or None)
        if self.streams:
            cur = _stream().value
            for a in self.streams:
                a.value = cur
        for fn, args, what, kernels in self.calls:
            _check(_launch(fn, *args), what, kernels)


_TAPE: Optional[LaunchTape] = None
TAPE_REPEATS = 0            # tapes repeated since this was last set to 0
REPEAT_LAYERS = True        # whether a model repeats the recorded launches of equal blocks (engine/model.py)


def _launch(fn, *args) -> int:
    """Every kernel launch of this module goes through here."""
    if _TAPE is not None:
        _TAPE.calls.append([fn, args, None, 1])
    return fn(*args)


def empty(shape, dtype, device) -> torch.Tensor:
    """Uninitialised memory for a kernel's output (what the kernels' callers allocate with, so that a
    tape of launches can keep it)."""
    t = torch.empty(shape, dtype=dtype, device=device)
    if _TAPE is not None:
        _TAPE.temps.append(t)
    return t


def dtype_code(t: torch.dtype) -> int:
    if t == torch.float32:
        return F32
    if t == torch.bfloat16:
        return BF16
    raise KernelError(f"element type {t} is not supported by the kernels (float32 and bfloat16 are)")


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> "_StreamArg":
    # (the raw handle straight from the runtime: a step launches a few hundred kernels, and building a
    # Stream object for each costs more host time than a short kernel runs)
    if _RAW_STREAM is not None:
        return _StreamArg(_RAW_STREAM(torch.cuda.current_device()))
    return _StreamArg(torch.cuda.current_stream().cuda_stream)


def _ptr(t: Optional[torch.Tensor]) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _addr(t: Optional[torch.Tensor]):
    """Address for a structure field (None is a null pointer)."""
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor: the kernels have no CPU path")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, is {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise KernelError(f"{name} must have shape {tuple(shape)}, has {tuple(t.shape)}")


_LIBS: dict = {}
# GOPHERLLM_DEBUG_BOUNDS=1 selects builds of the kernels that check the indices they take from memory
# (token ids, page numbers, positions) and record a bad one instead of using it; see bounds_status().
DEBUG_BOUNDS = os.environ.get("GOPHERLLM_DEBUG_BOUNDS", "") not in ("", "0")


def _lib(source: str, defines=()):
    if DEBUG_BOUNDS:
        defines = tuple(defines) + ("GL_DEBUG_BOUNDS=1",)
    key = (source, tuple(defines))
    lib = _LIBS.get(key)
    if lib is None:
        lib = _LIBS[key] = build.load(source, key[1])
    return lib


# ---------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, scale: float = 1.0,
          out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[t] = scale * table[tokens[t]] as float32."""
    _need(table, "table")
    _need(tokens, "tokens", torch.int32)
    V, D = table.shape
    T = tokens.numel()
    if out is None:
        out = empty((T, D), torch.float32, table.device)
    _need(out, "out", torch.float32, (T, D))
    fn = _lib("rowwise.cu").gl_embed
    _check(_launch(fn, _ptr(table), c_int(dtype_code(table.dtype)), _ptr(tokens), _ptr(out),
              c_int(T), c_int(D), c_int(V), c_float(scale), _stream()), "embed")
    return out


def add_rows(table: torch.Tensor, index: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] += table[index[t]] (float32 rows; a table of learned positions added to the residual stream)."""
    _need(table, "table")
    _need(index, "index", torch.int32)
    N, D = table.shape
    _need(out, "out", torch.float32, (index.numel(), D))
    fn = _lib("rowwise.cu").gl_add_rows
    _check(_launch(fn, _ptr(table), c_int(dtype_code(table.dtype)), _ptr(index), _ptr(out),
              c_int(index.numel()), c_int(D), c_int(N), _stream()), "add_rows")
    return out


def scale_softcap(x: torch.Tensor, scale: float = 1.0, cap: float = 0.0) -> torch.Tensor:
    """In place on float32 logits: x * scale, then cap * tanh(x / cap) when cap > 0."""
    _need(x, "x", torch.float32)
    fn = _lib("rowwise.cu").gl_scale_softcap
    _check(_launch(fn, _ptr(x), ctypes.c_longlong(x.numel()), c_float(scale), c_float(cap), _stream()), "scale_softcap")
    return x


def norm(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], eps: float,
         out_dtype: torch.dtype, rms: bool = False, rows: Optional[torch.Tensor] = None,
         out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """LayerNorm (or RMSNorm) of float32 rows; ``rows`` picks rows of x."""
    _need(x, "x", torch.float32)
    D = x.shape[-1]
    _need(gamma, "gamma", torch.float32, (D,))
    if beta is not None:
        _need(beta, "beta", torch.float32, (D,))
    if rows is not None:
        _need(rows, "rows", torch.int32)
        R = rows.numel()
    else:
        R = x.numel() // D
    if out is None:
        out = empty((R, D), out_dtype, x.device)
    _need(out, "out", out_dtype, (R, D))
    fn = _lib("rowwise.cu").gl_norm
    _check(_launch(fn, _ptr(x), _ptr(rows), _ptr(gamma), _ptr(beta), _ptr(out), c_int(dtype_code(out_dtype)),
              c_int(R), c_int(D), c_float(eps), c_int(1 if rms else 0), _stream()), "norm")
    return out


def advance_decode(tokens, tok_pos, seq_ctx, sampled, history, counter) -> None:
    """After a decode step on the device: tokens <- sampled, positions and cached lengths + 1,
    history[counter] <- sampled, counter + 1 (all int32; history is [max_steps, B])."""
    B = tokens.numel()
    for n, t in (("tokens", tokens), ("tok_pos", tok_pos), ("seq_ctx", seq_ctx)):
        _need(t, n, torch.int32, (B,))
    _need(sampled, "sampled", torch.int32)
    _need(history, "history", torch.int32)
    _need(counter, "counter", torch.int32, (1,))
    if sampled.numel() < B or history.shape[-1] != B:
        raise KernelError("advance_decode: sampled or history does not match the batch")
    fn = _lib("rowwise.cu").gl_advance_decode
    _check(_launch(fn, _ptr(tokens), _ptr(tok_pos), _ptr(seq_ctx), _ptr(sampled), _ptr(history), _ptr(counter),
              c_int(B), c_int(history.shape[0]), _stream()), "advance_decode")


def rope_table(pos: torch.Tensor, inv_freq: torch.Tensor):
    """cos and sin of float32(pos) * inv_freq, each [T, half] float32."""
    _need(pos, "pos", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    T, half = pos.numel(), inv_freq.numel()
    cosv = empty((T, half), torch.float32, pos.device)
    sinv = empty(cosv.shape, cosv.dtype, cosv.device)
    fn = _lib("qkv_cache.cu").gl_rope_table
    _check(_launch(fn, _ptr(pos), _ptr(inv_freq), _ptr(cosv), _ptr(sinv), c_int(T), c_int(half), _stream()),
           "rope_table")
    return cosv, sinv


class _QkvCacheArgs(Structure):
    _fields_ = [("qkv", c_void_p), ("q_out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("cosv", c_void_p), ("sinv", c_void_p),
                ("q_gamma", c_void_p), ("q_beta", c_void_p), ("k_gamma", c_void_p), ("k_beta", c_void_p),
                ("tok_seq", c_void_p), ("tok_pos", c_void_p), ("pages", c_void_p),
                ("T", c_int), ("nH", c_int), ("nKV", c_int), ("hd", c_int), ("half", c_int),
                ("max_pages", c_int), ("interleaved", c_int), ("norm_rms", c_int), ("write_kv", c_int),
                ("eps", c_float), ("q_scale", c_float), ("n_pages", c_int)]


def qkv_to_cache(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 tok_seq: torch.Tensor, tok_pos: torch.Tensor, pages: torch.Tensor,
                 num_heads: int, num_kv_heads: int, head_dim: int, q_scale: float,
                 cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                 interleaved: bool = False,
                 q_norm=None, k_norm=None, norm_eps: float = 0.0, norm_rms: bool = False,
                 write_kv: bool = True) -> None:
    """Head norm, rotation and scale of projected rows; q to ``q_out``, k and v into cache pages.

    qkv: [T, (nH + 2 nKV) * hd]; k_cache, v_cache: [pages, nKV, PAGE, hd];
    pages: [B, max_pages] int32; q_norm / k_norm: (gamma, beta or None) or None.
    """
    _need(qkv, "qkv")
    T = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    _need(qkv, "qkv", shape=(T, width))
    _need(q_out, "q_out", qkv.dtype, (T, num_heads * head_dim))
    _need(k_cache, "k_cache")
    _need(v_cache, "v_cache", k_cache.dtype, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    _need(tok_seq, "tok_seq", torch.int32, (T,))
    _need(tok_pos, "tok_pos", torch.int32, (T,))
    _need(pages, "pages", torch.int32)
    half = 0
    if cos is not None:
        half = cos.shape[-1]
        _need(cos, "cos", torch.float32, (T, half))
        _need(sin, "sin", torch.float32, (T, half))
        if 2 * half > head_dim:
            raise KernelError(f"rotary dimension {2 * half} exceeds head size {head_dim}")
    qg = qb = kg = kb = None
    if q_norm is not None:
        qg, qb = q_norm
        kg, kb = k_norm
        for n, t in (("q_norm.gamma", qg), ("k_norm.gamma", kg)):
            _need(t, n, torch.float32, (head_dim,))
        for n, t in (("q_norm.beta", qb), ("k_norm.beta", kb)):
            if t is not None:
                _need(t, n, torch.float32, (head_dim,))
    a = _QkvCacheArgs(qkv.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                      _addr(cos), _addr(sin), _addr(qg), _addr(qb), _addr(kg), _addr(kb),
                      tok_seq.data_ptr(), tok_pos.data_ptr(), pages.data_ptr(),
                      T, num_heads, num_kv_heads, head_dim, half, pages.shape[-1],
                      1 if interleaved else 0, 1 if norm_rms else 0, 1 if write_kv else 0,
                      norm_eps, q_scale, k_cache.shape[0])
    fn = _lib("qkv_cache.cu").gl_qkv_cache
    _check(_launch(fn, byref(a), c_int(dtype_code(qkv.dtype)), c_int(dtype_code(k_cache.dtype)), _stream()),
           "qkv_to_cache")


class _AttnArgs(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("seq_qstart", c_void_p), ("seq_qlen", c_void_p), ("seq_ctx", c_void_p), ("pages", c_void_p),
                ("B", c_int), ("nH", c_int), ("nKV", c_int), ("hd", c_int), ("max_pages", c_int),
                ("window", c_int), ("max_qlen", c_int), ("score_scale", c_float),
                # (appended: the kernels that check indices read it, the others' records end before it)
                ("n_pages", c_int)]


def _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
               num_heads, num_kv_heads, head_dim, window, max_qlen, score_scale) -> _AttnArgs:
    T = q.shape[0]
    _need(q, "q", shape=(T, num_heads * head_dim))
    _need(out, "out", q.dtype, q.shape)
    _need(k_cache, "k_cache")
    _need(v_cache, "v_cache", k_cache.dtype, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    B = seq_qlen.numel()
    for n, t in (("seq_qstart", seq_qstart), ("seq_qlen", seq_qlen), ("seq_ctx", seq_ctx)):
        _need(t, n, torch.int32, (B,))
    _need(pages, "pages", torch.int32)
    if pages.shape[0] != B:
        raise KernelError(f"pages has {pages.shape[0]} rows for {B} sequences")
    if num_heads % num_kv_heads:
        raise KernelError(f"{num_heads} heads are not a multiple of {num_kv_heads} key/value heads")
    return _AttnArgs(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                     seq_qstart.data_ptr(), seq_qlen.data_ptr(), seq_ctx.data_ptr(), pages.data_ptr(),
                     B, num_heads, num_kv_heads, head_dim, pages.shape[-1], window, max_qlen, score_scale,
                     k_cache.shape[0])


def attention_generic(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                      num_heads: int, num_kv_heads: int, head_dim: int, max_qlen: int,
                      window: int = 0, score_scale: float = 1.0) -> None:
    """Causal attention of this step's queries over the paged cache, 32-bit arithmetic."""
    if head_dim > 256:
        raise KernelError(f"head size {head_dim} exceeds 256")
    a = _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                   num_heads, num_kv_heads, head_dim, window, max_qlen, score_scale)
    fn = _lib("attention_generic.cu").gl_attention_generic
    _check(_launch(fn, byref(a), c_int(dtype_code(q.dtype)), c_int(dtype_code(k_cache.dtype)), _stream()),
           "attention_generic")


def attention_prefill(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                      num_heads: int, num_kv_heads: int, head_dim: int, max_qlen: int,
                      window: int = 0) -> None:
    """Causal attention of runs of new tokens over the bfloat16 cache on tensor cores
    (mma.sync, 32-bit softmax); head sizes 16..256 in steps of 16."""
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"prefill attention takes head sizes 16..256 in steps of 16, not {head_dim}")
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError("prefill attention takes bfloat16 queries and cache")
    a = _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                   num_heads, num_kv_heads, head_dim, window, max_qlen, 1.0)
    lib = _lib("attention_prefill.cu", catalog.head_dim_defines(head_dim))
    _check(_launch(lib.gl_attention_prefill, byref(a), _stream()), "attention_prefill")


def attention_prefill_tc(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                         num_heads: int, num_kv_heads: int, head_dim: int, max_qlen: int,
                         window: int = 0) -> None:
    """Causal attention of runs of new tokens over the bfloat16 cache on the 5th-generation
    tensor cores (tcgen05.mma for both products, operands by TMA, scores and partial outputs
    in tensor memory); head sizes 16..128 in steps of 16."""
    if head_dim % 16 or not 16 <= head_dim <= 128:
        raise KernelError(f"tcgen05 prefill attention takes head sizes 16..128 in steps of 16, not {head_dim}")
    if q.dtype != torch.bfloat16 or k_cache.dtype != torch.bfloat16:
        raise KernelError("prefill attention takes bfloat16 queries and cache")
    a = _attn_args(q, out, k_cache, v_cache, seq_qstart, seq_qlen, seq_ctx, pages,
                   num_heads, num_kv_heads, head_dim, window, max_qlen, 1.0)
    lib = _lib("attention_prefill_tc.cu", catalog.head_dim_defines(head_dim))
    _check(_launch(lib.gl_attention_prefill_tc, byref(a), c_int(q.shape[0]), c_int(k_cache.shape[0]), _stream()),
           "attention_prefill_tc")


class _DecodeArgs(Structure):
    _fields_ = [("q", c_void_p), ("out", c_void_p), ("k_cache", c_void_p), ("v_cache", c_void_p),
                ("seq_ctx", c_void_p), ("pages", c_void_p), ("part_o", c_void_p), ("part_ml", c_void_p),
                ("B", c_int), ("nH", c_int), ("nKV", c_int), ("max_pages", c_int), ("window", c_int),
                ("splits", c_int)]


class _DecodeQkv(Structure):
    _fields_ = [("qkv", c_void_p), ("cosv", c_void_p), ("sinv", c_void_p), ("half", c_int), ("write_kv", c_int),
                ("q_scale", c_float)]


DECODE_MAX_GROUP = 8      # query heads per key/value head the decode kernel takes
_SM_COUNT = {}


def sm_count(device) -> int:
    idx = torch.device(device).index or 0
    if idx not in _SM_COUNT:
        _SM_COUNT[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    return _SM_COUNT[idx]


def decode_blocks_per_sm(head_dim: int, group: int = 1) -> int:
    """Blocks of the decode kernel one SM holds at once (bounded by shared memory)."""
    stages = 2
    smem = 2 * stages * PAGE * (2 * head_dim + 16) + 1024 + 4 * (64 + 5 * head_dim * max(1, group) + 16)
    return max(1, min(8, (227 * 1024) // (smem + 1024)))


def decode_splits(batch: int, num_kv_heads: int, max_len: int, device, head_dim: int,
                  group: int = 1) -> int:
    """How many blocks share one (sequence, key/value head).  Never more blocks than are resident
    at once (a grid a little larger than the machine would run a second, nearly empty wave), never
    more than the longest sequence has pages.  Within that: enough blocks to put about 1.7 on every
    SM, and enough that a block has at most 8 pages to walk through; more blocks than that only
    take the SMs' shared memory from the products that run beside a short attention.  Measured on
    Phi-2 shapes (32 heads of 80, 148 SMs; batches of 2 to 8, 512 to 2,048 positions) this is
    within 3 % of the best split everywhere and up to 11 % a step better than filling every slot."""
    pages = max(1, -(-max_len // PAGE))
    sms = sm_count(device)
    per = max(1, batch * num_kv_heads)
    slots = sms * decode_blocks_per_sm(head_dim, group)
    want = max(-(-(17 * sms // 10) // per), -(-pages // 8))
    return max(1, min(want, slots // per, pages, 8))


def decode_takes_qkv(act_dtype, cache_dtype, head_dim: int, rotary_half: int, interleaved: bool,
                     head_norm: bool) -> bool:
    """Whether decode attention can take the projection's output itself (rotating and scaling the
    queries, rotating and storing the new key and value) instead of a pass of qkv_to_cache first."""
    return (act_dtype == torch.bfloat16 and cache_dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 256
            and rotary_half % 8 == 0 and not interleaved and not head_norm)


def attention_decode(q, out, k_cache, v_cache, seq_ctx, pages, num_heads: int, num_kv_heads: int,
                     head_dim: int, splits: int, window: int = 0,
                     scratch: Optional[torch.Tensor] = None, qkv: Optional[torch.Tensor] = None,
                     cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                     q_scale: float = 1.0, write_kv: bool = True) -> None:
    """One query per sequence (row b of q is sequence b) over the bfloat16 cache.
    Up to 8 splits merge inside a thread-block cluster and need no scratch.  More splits, or
    ``scratch`` given (float32, at least B*nH*splits*(hd+2) elements), write partial results
    to scratch (allocated here when needed and not given) for a second kernel to merge.
    With ``qkv`` ([B, (heads + 2 kv heads) * head size], the projection's output; q is None then)
    the kernel rotates (cos, sin: [B, half] float32, split-half pairing) and scales the queries itself,
    and stores the new token's rotated key and its value in the cache (write_kv) before it reads them."""
    B = out.shape[0]
    if qkv is not None:
        _need(qkv, "qkv", torch.bfloat16, (B, (num_heads + 2 * num_kv_heads) * head_dim))
        half = 0
        if cos is not None:
            _need(cos, "cos", torch.float32)
            _need(sin, "sin", torch.float32, cos.shape)
            half = cos.shape[1]
            if cos.shape[0] != B or half % 8 or 2 * half > head_dim:
                raise KernelError(f"rotary tables {tuple(cos.shape)} do not fit {B} tokens of head size {head_dim}")
    else:
        _need(q, "q", torch.bfloat16, (B, num_heads * head_dim))
    _need(out, "out", torch.bfloat16, (B, num_heads * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    _need(seq_ctx, "seq_ctx", torch.int32, (B,))
    _need(pages, "pages", torch.int32)
    if pages.shape[0] != B:
        raise KernelError(f"pages has {pages.shape[0]} rows for {B} sequences")
    if head_dim % 16 or not 16 <= head_dim <= 256:
        raise KernelError(f"decode attention takes head sizes 16..256 in steps of 16, not {head_dim}")
    if num_heads % num_kv_heads or num_heads // num_kv_heads > DECODE_MAX_GROUP:
        raise KernelError(f"decode attention takes up to {DECODE_MAX_GROUP} query heads per key/value head")
    lib = _lib("attention_decode.cu", catalog.head_dim_defines(head_dim))
    part_o = part_ml = None
    if splits > 8 or (splits > 1 and scratch is not None):
        n_o, n_ml = B * num_heads * splits * head_dim, B * num_heads * splits * 2
        if scratch is None:
            scratch = empty(n_o + n_ml, torch.float32, out.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < n_o + n_ml:
            raise KernelError("decode attention scratch is too small")
        part_o, part_ml = scratch.data_ptr(), scratch.data_ptr() + 4 * n_o
    a = _DecodeArgs(_addr(q), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                    seq_ctx.data_ptr(), pages.data_ptr(), part_o, part_ml,
                    B, num_heads, num_kv_heads, pages.shape[-1], window, splits)
    launches = 2 if part_o is not None else 1
    if qkv is None:
        _check(_launch(lib.gl_attention_decode, byref(a), _stream()), "attention_decode", launches)
    else:
        x = _DecodeQkv(qkv.data_ptr(), _addr(cos), _addr(sin), cos.shape[1] if cos is not None else 0,
                       int(bool(write_kv)), float(q_scale))
        _check(_launch(lib.gl_attention_decode_qkv, byref(a), byref(x), _stream()), "attention_decode", launches)


def attention(q, out, k_cache, v_cache, ctx, pages, num_heads: int, num_kv_heads: int,
              head_dim: int, window: int = 0) -> None:
    """Attention of a step's queries over the cache with the fastest kernel for the step's
    shape and element type.  ``ctx`` is the step's context (per-sequence starts, lengths,
    cached lengths on the device; the longest query run and sequence on the host)."""
    if (ctx.is_decode and q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16
            and head_dim % 16 == 0 and num_heads // num_kv_heads <= DECODE_MAX_GROUP):
        splits = decode_splits(ctx.n_seqs, num_kv_heads, ctx.max_len, q.device, head_dim,
                               num_heads // num_kv_heads)
        attention_decode(q, out, k_cache, v_cache, ctx.seq_ctx, pages, num_heads, num_kv_heads,
                         head_dim, splits, window)
        return
    if q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and head_dim % 16 == 0:
        if USE_TCGEN05 and head_dim <= TC_ATTENTION_MAX_HEAD_DIM:
            attention_prefill_tc(q, out, k_cache, v_cache, ctx.seq_qstart, ctx.seq_qlen, ctx.seq_ctx, pages,
                                 num_heads, num_kv_heads, head_dim, ctx.max_qlen, window)
            return
        attention_prefill(q, out, k_cache, v_cache, ctx.seq_qstart, ctx.seq_qlen, ctx.seq_ctx, pages,
                          num_heads, num_kv_heads, head_dim, ctx.max_qlen, window)
        return
    attention_generic(q, out, k_cache, v_cache, ctx.seq_qstart, ctx.seq_qlen, ctx.seq_ctx, pages,
                      num_heads, num_kv_heads, head_dim, ctx.max_qlen, window)


class _DecodeLayerArgs(Structure):
    _fields_ = [("x", c_void_p), ("norm_g", c_void_p), ("norm_b", c_void_p),
                ("w_qkv", c_void_p), ("b_qkv", c_void_p), ("w_up", c_void_p), ("b_up", c_void_p),
                ("w_out", c_void_p), ("b_out", c_void_p), ("w_down", c_void_p), ("b_down", c_void_p),
                ("k_cache", c_void_p), ("v_cache", c_void_p), ("pages", c_void_p), ("seq_ctx", c_void_p),
                ("cosv", c_void_p), ("sinv", c_void_p),
                ("xn", c_void_p), ("qkv", c_void_p), ("o", c_void_p), ("h", c_void_p),
                ("scratch", c_void_p), ("sync", c_void_p),
                ("M", c_int), ("D", c_int), ("I", c_int), ("nH", c_int), ("nKV", c_int), ("half", c_int),
                ("max_pages", c_int), ("n_pages", c_int), ("window", c_int), ("act", c_int), ("rms", c_int),
                ("write_kv", c_int), ("eps", c_float), ("q_scale", c_float)]


DECODE_LAYER_MAX_ROWS = 64
# Fewer tokens than this go through the separate kernels, which are faster there.  Measured on Phi-2's
# sizes, ms a step of 32 layers, separate kernels against the fused layer: 1 token 1.40 / 1.82, 8 tokens
# 1.92 / 2.21, 16 tokens 2.46 / 2.72, 17 tokens 2.83 / 2.79, 32 tokens 3.81 / 3.61 (1,024 positions each);
# 64 tokens of 128 positions 3.54 / 2.69, of 300 4.48 / 3.50, of 2,048 9.60 / 8.46.
DECODE_LAYER_MIN_ROWS = 17
# ... where the first products' 128-row tiles nearly fill the SMs one to a block (Phi-2: 140 tiles on 148
# SMs).  Where they do not (Phi-1.5: 112 tiles), part of the machine idles through that phase and the separate
# kernels stay ahead up to 32 tokens (Phi-1.5's sizes, 1,024 positions, separate / fused: 17 tokens 1.68 / 1.80,
# 24 tokens 1.94 / 2.08, 32 tokens 2.27 / 2.28, 33 tokens 2.68 / 2.39, 48 tokens 3.07 / 2.87, 64 tokens of
# 2,048 positions 5.57 / 5.15).
DECODE_LAYER_MIN_ROWS_CUT_TILES = 33
# ... and steps whose longest sequence is shorter than this (none: the fused layer is ahead at every
# context length from 17 tokens on).
DECODE_LAYER_MIN_CONTEXT = 0
DECODE_LAYER_MAX_HEAD_DIM = catalog.MAX_HEAD_DIM["decode_layer.cu"]
USE_DECODE_LAYER = True
_DECODE_LAYER_KEEP = None          # a dict here receives the work buffers of the last call (for tests)
_DECODE_LAYER_SYNC: dict = {}      # device index -> the int32 words the fused layer's blocks meet through


def decode_layer_takes(x, w_qkv, w_up, w_out, w_down, cache_dtype, head_dim: int, group: int, rotary_half: int,
                       interleaved: bool, head_norm: bool, longest: int = 1 << 30) -> bool:
    """Whether the fused decode layer takes these types and sizes (the caller falls back to the separate
    kernels otherwise): bfloat16 weights and cache, DECODE_LAYER_MIN_ROWS (or, where the first products' tiles do
    not fill the SMs one to a block, DECODE_LAYER_MIN_ROWS_CUT_TILES) to 64 tokens, a longest sequence
    (``longest``, positions after the step) of at least DECODE_LAYER_MIN_CONTEXT, head sizes up to 128 in steps of 16,
    up to 8 query heads per key/value head, split-half rotation over a multiple of 16 dims, no per-head
    norm, widths that are multiples of 8."""
    tiles = -(-w_qkv.shape[0] // 128) + -(-w_up.shape[0] // 128)
    blocks = sm_count(x.device)
    whole_tiles = tiles * 10 >= blocks * -(-tiles // blocks) * 9
    fewest = DECODE_LAYER_MIN_ROWS if whole_tiles else max(DECODE_LAYER_MIN_ROWS, DECODE_LAYER_MIN_ROWS_CUT_TILES)
    return (USE_DECODE_LAYER and fewest <= x.shape[0] <= DECODE_LAYER_MAX_ROWS
            and longest >= DECODE_LAYER_MIN_CONTEXT and cache_dtype == torch.bfloat16
            and all(w.dtype == torch.bfloat16 for w in (w_qkv, w_up, w_out, w_down))
            and head_dim % 16 == 0 and head_dim <= DECODE_LAYER_MAX_HEAD_DIM and group <= DECODE_MAX_GROUP
            # (head sizes 32 and 96: rows of 64 and 192 bytes put four rows of an ldmatrix on the same banks and
            # are not swizzled by the kernel; the separate kernels take those)
            and (head_dim % 32 != 0 or head_dim % 64 == 0)
            and rotary_half % 8 == 0 and not interleaved and not head_norm
            and x.shape[1] % 8 == 0 and w_up.shape[0] % 8 == 0 and w_out.shape[1] % 8 == 0)


def decode_layer(x: torch.Tensor, norm_g: torch.Tensor, norm_b: Optional[torch.Tensor], eps: float, rms: bool,
                 w_qkv: torch.Tensor, b_qkv, w_up: torch.Tensor, b_up, act, w_out: torch.Tensor, b_out,
                 w_down: torch.Tensor, b_down, k_cache: torch.Tensor, v_cache: torch.Tensor,
                 seq_ctx: torch.Tensor, pages: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                 q_scale: float, cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                 window: int = 0, write_kv: bool = True) -> torch.Tensor:
    """One decode step of a parallel block in one kernel, x updated in place:
    n = norm(x); x += attention(n) · w_outᵀ + b_out + act(n · w_upᵀ + b_up) · w_downᵀ + b_down, with one
    token per sequence (row b of x is sequence b's new token at position seq_ctx[b]); the new token's
    rotated key and its value go into the cache (write_kv).  All calls on a device share a few words of
    synchronisation state: they must follow one another on a stream, never overlap."""
    M, D = x.shape
    _need(x, "x", torch.float32)
    _need(norm_g, "norm weight", torch.float32, (D,))
    if norm_b is not None:
        _need(norm_b, "norm bias", torch.float32, (D,))
    Nqkv, No, I = (num_heads + 2 * num_kv_heads) * head_dim, num_heads * head_dim, w_up.shape[0]
    _need(w_qkv, "w_qkv", torch.bfloat16, (Nqkv, D))
    _need(w_up, "w_up", torch.bfloat16, (I, D))
    _need(w_out, "w_out", torch.bfloat16, (D, No))
    _need(w_down, "w_down", torch.bfloat16, (D, I))
    for n, b, k in (("b_qkv", b_qkv, Nqkv), ("b_up", b_up, I), ("b_out", b_out, D), ("b_down", b_down, D)):
        if b is not None:
            _need(b, n, torch.float32, (k,))
    _need(k_cache, "k_cache", torch.bfloat16)
    _need(v_cache, "v_cache", torch.bfloat16, k_cache.shape)
    if tuple(k_cache.shape[1:]) != (num_kv_heads, PAGE, head_dim):
        raise KernelError(f"cache pages must be [*, {num_kv_heads}, {PAGE}, {head_dim}], are {tuple(k_cache.shape)}")
    _need(seq_ctx, "seq_ctx", torch.int32, (M,))
    _need(pages, "pages", torch.int32)
    if pages.shape[0] != M:
        raise KernelError(f"pages has {pages.shape[0]} rows for {M} sequences")
    half = 0
    if cos is not None:
        _need(cos, "cos", torch.float32)
        _need(sin, "sin", torch.float32, cos.shape)
        half = cos.shape[1]
        if cos.shape[0] != M:
            raise KernelError(f"rotary tables {tuple(cos.shape)} do not fit {M} tokens")
    if act not in ACTIVATIONS:
        raise KernelError(f"activation {act!r} unknown")
    if M > DECODE_LAYER_MAX_ROWS or head_dim % 16 or head_dim > DECODE_LAYER_MAX_HEAD_DIM:
        raise KernelError(f"the fused decode layer takes up to {DECODE_LAYER_MAX_ROWS} tokens and head sizes up to "
                          f"{DECODE_LAYER_MAX_HEAD_DIM} in steps of 16")
    dev = x.device
    lib = _lib("decode_layer.cu", catalog.head_dim_defines(head_dim))
    bf = torch.bfloat16
    xn = empty((M, D), bf, dev)
    qkv = empty((M, Nqkv), bf, dev)
    o = empty((M, No), bf, dev)
    h = empty((M, I), bf, dev)
    a = _DecodeLayerArgs(x.data_ptr(), norm_g.data_ptr(), _addr(norm_b), w_qkv.data_ptr(), _addr(b_qkv),
                         w_up.data_ptr(), _addr(b_up), w_out.data_ptr(), _addr(b_out), w_down.data_ptr(), _addr(b_down),
                         k_cache.data_ptr(), v_cache.data_ptr(), pages.data_ptr(), seq_ctx.data_ptr(),
                         _addr(cos), _addr(sin), xn.data_ptr(), qkv.data_ptr(), o.data_ptr(), h.data_ptr(), None, None,
                         M, D, I, num_heads, num_kv_heads, half, pages.shape[-1], k_cache.shape[0], window,
                         ACTIVATIONS[act], 1 if rms else 0, 1 if write_kv else 0, eps, q_scale)
    n_scratch, n_sync = ctypes.c_longlong(0), ctypes.c_longlong(0)
    _check(lib.gl_decode_layer_sizes(byref(a), byref(n_scratch), byref(n_sync)), "decode_layer", 0)
    idx = dev.index or 0
    sync = _DECODE_LAYER_SYNC.get(idx)
    if sync is None or sync.numel() < n_sync.value:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the fused decode layer's synchronisation words must exist before a capture: "
                              "run the step once outside it")
        # zero once; every call leaves the counters zero again (the generation word only ever grows)
        sync = _DECODE_LAYER_SYNC[idx] = torch.zeros(max(int(n_sync.value), 1 << 16), dtype=torch.int32, device=dev)
    scratch = empty(max(1, int(n_scratch.value)), torch.float32, dev)
    a.scratch, a.sync = scratch.data_ptr(), sync.data_ptr()
    _check(_launch(lib.gl_decode_layer, byref(a), _stream()), "decode_layer")
    if _DECODE_LAYER_KEEP is not None:
        _DECODE_LAYER_KEEP.update(xn=xn, qkv=qkv, o=o, h=h)
    return x


def reset_decode_layer_sync() -> None:
    """Zero the fused decode layer's synchronisation words (after a kernel gave up a wait mid-way they
    may be left counting)."""
    for t in _DECODE_LAYER_SYNC.values():
        t.zero_()


class _GemmArgs(Structure):
    _fields_ = [("a", c_void_p), ("w", c_void_p), ("bias", c_void_p), ("add0", c_void_p),
                ("add1", c_void_p), ("out", c_void_p),
                ("M", c_int), ("N", c_int), ("K", c_int), ("act", c_int),
                # a second product summed into the same output (the tcgen05 kernel reads these; the
                # other kernels' argument structs end before them)
                ("a2", c_void_p), ("w2", c_void_p), ("bias2", c_void_p), ("K2", c_int),
                # a second set of columns from the same rows (tcgen05 kernel only)
                ("wB", c_void_p), ("biasB", c_void_p), ("outB", c_void_p), ("NB", c_int), ("actB", c_int)]


def _gemm_args(a, w, bias, act, add0, add1, out) -> _GemmArgs:
    _need(a, "a")
    _need(w, "w")
    M, K = a.shape
    N = w.shape[0]
    if w.shape[1] != K:
        raise KernelError(f"a is [{M}, {K}] but w is {tuple(w.shape)}")
    if bias is not None:
        _need(bias, "bias", torch.float32, (N,))
    for n, t in (("add0", add0), ("add1", add1)):
        if t is not None:
            _need(t, n, torch.float32, (M, N))
    _need(out, "out", shape=(M, N))
    if act not in ACTIVATIONS:
        raise KernelError(f"activation {act!r} unknown")
    return _GemmArgs(a.data_ptr(), w.data_ptr(), _addr(bias), _addr(add0), _addr(add1), out.data_ptr(),
                     M, N, K, ACTIVATIONS[act], None, None, None, 0, None, None, None, 0, 0)


def gemm_simt(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
              add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
              out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(a · wᵀ + bias) + add0 + add1 on CUDA cores in 32-bit (any element type, any size)."""
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    fn = _lib("gemm_simt.cu").gl_gemm_simt
    _check(_launch(fn, byref(g), c_int(dtype_code(a.dtype)), c_int(dtype_code(w.dtype)),
              c_int(dtype_code(out.dtype)), _stream()), "gemm_simt")
    return out


SKINNY_MAX_ROWS = 64
USE_TCGEN05 = True
TC_ATTENTION_MAX_HEAD_DIM = catalog.MAX_HEAD_DIM["attention_prefill_tc.cu"]


def gemm_tcgen05_cut_tiles(mode: int) -> None:
    """How the tcgen05 product shares work when it adds onto its output: 0 whole tiles (default),
    1 equal shares of (tile, k-block) units whenever possible, -1 shares only when whole tiles would
    fill the SMs unevenly."""
    _lib("gemm_tcgen05.cu").gl_gemm_tcgen05_set_split(c_int(mode))


def _second_product(g: _GemmArgs, a, w, second) -> None:
    """Fill in the operands of a second product summed into the same output."""
    a2, w2, bias2 = second
    _need(a2, "a2", torch.bfloat16)
    _need(w2, "w2", torch.bfloat16)
    if a2.shape[0] != a.shape[0] or w2.shape[0] != w.shape[0] or a2.shape[1] != w2.shape[1] or a2.shape[1] % 8:
        raise KernelError(f"second product [{tuple(a2.shape)}] x [{tuple(w2.shape)}] does not fit the first")
    if bias2 is not None:
        _need(bias2, "bias2", torch.float32, (w.shape[0],))
    g.a2, g.w2, g.bias2, g.K2 = a2.data_ptr(), w2.data_ptr(), _addr(bias2), a2.shape[1]


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
                add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                split_k: int = 0, second=None) -> torch.Tensor:
    """The weight-streaming product for up to 64 rows of bfloat16 activations (K a multiple of 8).
    ``second`` = (a2, w2, bias2) sums another product into the same output (K a multiple of 64 then)."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    if a.shape[0] > SKINNY_MAX_ROWS or a.shape[1] % 8:
        raise KernelError(f"gemm_skinny takes up to {SKINNY_MAX_ROWS} rows and K a multiple of 8")
    if second is not None:
        if a.shape[1] % 64:
            raise KernelError("gemm_skinny takes a second product only behind a K that is a multiple of 64")
        _second_product(g, a, w, second)
    fn = _lib("gemm_skinny.cu").gl_gemm_skinny
    _check(_launch(fn, byref(g), c_int(dtype_code(out.dtype)), c_int(split_k), _stream()), "gemm_skinny")
    return out


STREAM_MIN_ROWS, STREAM_MAX_ROWS = 17, 64
# Off: as measured with Phi-2's sizes the mma.sync product is as fast or faster at 17 to 64 rows (64 rows:
# 19.5 / 29.8 / 39.9 µs for the qkv, the up and the joined out+down product against 19.8 / 25.7 / 25.7),
# both far from the weights' streaming time; what a block pays once (tensor-memory allocation, two cluster
# barriers, the reduction through the peers' shared memory) stands against ten to twenty stages of work.
USE_GEMM_STREAM = False


def gemm_stream(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
                add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
                out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                split_k: int = 0, second=None) -> torch.Tensor:
    """The weight-streaming product for up to 64 rows on the 5th-generation tensor cores: the weights
    are the 128-row operand of tcgen05.mma, the tokens its N (K a multiple of 8).  Meant for 17 to 64
    rows, where the tokens' tile is too large to be fetched again for every 64 weight rows.
    ``second`` = (a2, w2, bias2) sums another product into the same output (K a multiple of 64 then)."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    if a.shape[0] > STREAM_MAX_ROWS or a.shape[1] % 8:
        raise KernelError(f"gemm_stream takes up to {STREAM_MAX_ROWS} rows and K a multiple of 8")
    if second is not None:
        if a.shape[1] % 64:
            raise KernelError("gemm_stream takes a second product only behind a K that is a multiple of 64")
        _second_product(g, a, w, second)
    fn = _lib("gemm_stream.cu").gl_gemm_stream
    _check(_launch(fn, byref(g), c_int(dtype_code(out.dtype)), c_int(split_k), _stream()), "gemm_stream")
    return out


def _few_rows(a, w, bias, act, add0, add1, out_dtype, out, second=None):
    """The weight-streaming product for up to 64 rows: mma.sync for up to 16, tcgen05 above."""
    if USE_GEMM_STREAM and a.shape[0] >= STREAM_MIN_ROWS:
        return gemm_stream(a, w, bias, act, add0, add1, out_dtype, out, second=second)
    return gemm_skinny(a, w, bias, act, add0, add1, out_dtype, out, second=second)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
                 add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
                 out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None,
                 tile_n: int = 0, _defines=(), second=None, fork=None):
    """The tensor-core product (tcgen05.mma fed by TMA, accumulators in tensor memory) for
    bfloat16 operands with K a multiple of 8; meant for many rows.  ``second`` = (a2, w2, bias2)
    sums another product over the same rows and columns into the tile before the epilogue:
    out = act(a·wᵀ + a2·w2ᵀ + bias + bias2) + add0 + add1.  ``fork`` = (wB, biasB, actB) computes a
    second output actB(a·wBᵀ + biasB) in the same launch (nothing added, no ``second``; both
    outputs' rows whole 16-byte units) and makes the result the pair (out, outB)."""
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16)
    if out is None:
        out = empty((a.shape[0], w.shape[0]), out_dtype or a.dtype, a.device)
    g = _gemm_args(a, w, bias, act, add0, add1, out)
    if a.shape[1] % 8:
        raise KernelError("gemm_tcgen05 takes K a multiple of 8 (TMA needs 16-byte row pitch)")
    if second is not None:
        _second_product(g, a, w, second)
    out_b = None
    if fork is not None:
        w_b, bias_b, act_b = fork
        _need(w_b, "wB", torch.bfloat16)
        if w_b.shape[1] != a.shape[1] or act_b not in ACTIVATIONS:
            raise KernelError(f"second set of columns {tuple(w_b.shape)} does not fit a {tuple(a.shape)}")
        if bias_b is not None:
            _need(bias_b, "biasB", torch.float32, (w_b.shape[0],))
        out_b = empty((a.shape[0], w_b.shape[0]), out.dtype, a.device)
        g.wB, g.biasB, g.outB, g.NB, g.actB = w_b.data_ptr(), _addr(bias_b), out_b.data_ptr(), w_b.shape[0], ACTIVATIONS[act_b]
    if tile_n not in (0, 64, 128, 160, 192, 256, 1160, 1192, 1256):
        raise KernelError("tile_n is 0 (choose), 64, 128, 160 (32-bit output only), 192 or 256; "
                          "1000 more for tiles of 256 rows (160, 192, 256)")
    fn = _lib("gemm_tcgen05.cu", _defines).gl_gemm_tcgen05
    _check(_launch(fn, byref(g), c_int(dtype_code(out.dtype)), c_int(tile_n), _stream()), "gemm_tcgen05")
    return out if fork is None else (out, out_b)


def wait_failures(clear: bool = False) -> dict:
    """Which of the loaded libraries recorded a bounded wait that ran out (what they computed since is
    invalid): library name -> 1, 0, or -1 if the word could not be read.  ``clear`` sets the words back
    to 0.  Reading a word waits for the device."""
    out = {}
    for key, lib in list(build._loaded.items()):
        if hasattr(lib, "gl_wait_status"):
            out[key] = int(lib.gl_wait_status(c_int(1 if clear else 0)))
    return out


_BOUNDS_KINDS = {1: "token id", 2: "page number", 3: "position in a page table", 4: "row of a table"}


def bounds_status(clear: bool = False) -> dict:
    """In a build that checks indices (GOPHERLLM_DEBUG_BOUNDS=1): library name -> (kind, value, limit,
    count) of the bad indices its kernels met since the words were last cleared; libraries without
    violations are left out.  Empty in an ordinary build."""
    out = {}
    for key, lib in list(build._loaded.items()):
        if hasattr(lib, "gl_bounds_status"):
            words = (c_int * 4)()
            if lib.gl_bounds_status(words, c_int(1 if clear else 0)) != 0:
                out[key] = ("unreadable", 0, 0, 0)
            elif words[0] != 0:
                out[key] = (_BOUNDS_KINDS.get(words[0], str(words[0])), words[1], words[2], words[3])
    return out


def check_wait_failures() -> None:
    """Raise KernelError naming every library whose kernels gave up a bounded wait since the last
    check; the words are cleared, so the next check speaks of what ran after this one."""
    oob = bounds_status(clear=True)
    if oob:
        raise KernelError("kernels met indices outside their tables: " + "; ".join(
            f"{lib}: {kind} {value} (limit {limit}, {count} in all)" for lib, (kind, value, limit, count) in sorted(oob.items())))
    bad = sorted(k for k, v in wait_failures(clear=True).items() if v != 0)
    if bad:
        reset_decode_layer_sync()
        raise KernelError("a kernel gave up waiting (for a TMA copy or a tensor-core product) in "
                          + ", ".join(bad) + ": the results since the last check are invalid")


def linear_pair(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor],
                a2: torch.Tensor, w2: torch.Tensor, bias2: Optional[torch.Tensor],
                add0: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = a·wᵀ + bias + a2·w2ᵀ + bias2 + add0: the last products of two branches that are added
    to the same rows.  In bfloat16 both run as one product over the joined K (one kernel, one pass
    over the output); otherwise one after the other, each adding onto out."""
    if (a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a2.dtype == torch.bfloat16
            and w2.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and a2.shape[1] % 8 == 0):
        if a.shape[0] <= SKINNY_MAX_ROWS:
            if a.shape[1] % 64 == 0:
                return _few_rows(a, w, bias, None, add0, None, torch.float32, out, second=(a2, w2, bias2))
            if a2.shape[1] % 64 == 0:                  # the product whose K fills whole stages goes first
                return _few_rows(a2, w2, bias2, None, add0, None, torch.float32, out, second=(a, w, bias))
        elif USE_TCGEN05:
            return gemm_tcgen05(a, w, bias, None, add0, None, torch.float32, out, second=(a2, w2, bias2))
    out = linear(a, w, bias, add0=add0, out_dtype=torch.float32, out=out)
    return linear(a2, w2, bias2, add0=out, out=out)


def linear_fork(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], act,
                w_b: torch.Tensor, bias_b: Optional[torch.Tensor], act_b, out_dtype: Optional[torch.dtype] = None):
    """(act(a·wᵀ + bias), act_b(a·w_bᵀ + bias_b)): the first products of two branches that read the
    same rows.  For many rows of bfloat16 both run as one grid of tensor-core tiles; otherwise one
    after the other."""
    dt = out_dtype or a.dtype
    if (USE_TCGEN05 and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w_b.dtype == torch.bfloat16
            and a.shape[0] > SKINNY_MAX_ROWS and a.shape[1] % 8 == 0
            and (w.shape[0] * dt.itemsize) % 16 == 0 and (w_b.shape[0] * dt.itemsize) % 16 == 0):
        return gemm_tcgen05(a, w, bias, act, out_dtype=dt, fork=(w_b, bias_b, act_b))
    return linear(a, w, bias, act, out_dtype=dt), linear(a, w_b, bias_b, act_b, out_dtype=dt)


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
           add0: Optional[torch.Tensor] = None, add1: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out = act(a · wᵀ + bias) + add0 + add1 with the fastest kernel that takes these
    types and sizes.  float32 operands always run the 32-bit CUDA-core product."""
    if a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0:
        if a.shape[0] <= SKINNY_MAX_ROWS:
            return _few_rows(a, w, bias, act, add0, add1, out_dtype, out)
        if USE_TCGEN05:
            return gemm_tcgen05(a, w, bias, act, add0, add1, out_dtype, out)
    return gemm_simt(a, w, bias, act, add0, add1, out_dtype, out)


class _SampleArgs(Structure):
    _fields_ = [("logits", c_void_p), ("work", c_void_p), ("state_row", c_void_p), ("recent", c_void_p),
                ("recent_n", c_void_p), ("rng", c_void_p), ("out", c_void_p),
                ("sort_key", c_void_p), ("sort_idx", c_void_p),
                ("B", c_int), ("V", c_int), ("vpad", c_int), ("top_k", c_int),
                ("temperature", c_float), ("top_p", c_float), ("min_p", c_float),
                ("repeat_penalty", c_float)]


def check_sampler(temperature: float, top_k: int, top_p: float, min_p: float, vocab: int) -> None:
    """Raise if the kernel does not take this combination of options."""
    greedy = temperature < 1e-6 or top_k == 1
    if greedy:
        return
    whole = not (0 < top_k < vocab)
    if not whole and top_k > SAMPLE_KMAX:
        raise KernelError(f"top_k {top_k} exceeds {SAMPLE_KMAX} (top_k 0 or >= vocabulary samples the whole row)")


def needs_sort_scratch(temperature: float, top_k: int, top_p: float, min_p: float, vocab: int) -> bool:
    """Whether sampling needs sorting scratch: never (a nucleus or min-p cut with top-k off finds its
    boundary by a search over the weights' bits, not by sorting the row)."""
    return False


def sort_scratch_size(vocab: int) -> int:
    n = 1
    while n < vocab:
        n <<= 1
    return n


def sample(logits: torch.Tensor, work: torch.Tensor, recent: torch.Tensor, recent_n: torch.Tensor,
           rng: torch.Tensor, out: torch.Tensor, temperature: float, top_k: int, top_p: float,
           min_p: float, repeat_penalty: float, state_row: Optional[torch.Tensor] = None,
           sort_key: Optional[torch.Tensor] = None, sort_idx: Optional[torch.Tensor] = None) -> None:
    """One token per row of float32 logits [B, V] into ``out`` [B] int32.

    recent [R, 64] int32 / recent_n [R] int32: each state row's window of recent tokens
    (the choice is appended); rng [R] int64: xorshift64 states; state_row [B] int32 says
    which state row a logits row uses (None: row b uses state b)."""
    _need(logits, "logits", torch.float32)
    B, V = logits.shape
    _need(work, "work", torch.float32)
    if work.numel() < B * V:
        raise KernelError("sampling scratch is smaller than the logits")
    R = recent_n.numel()
    _need(recent, "recent", torch.int32, (R, SAMPLE_WINDOW))
    _need(recent_n, "recent_n", torch.int32, (R,))
    _need(rng, "rng", torch.int64, (R,))
    _need(out, "out", torch.int32)
    if out.numel() < B:
        raise KernelError("out is smaller than the batch")
    if state_row is not None:
        _need(state_row, "state_row", torch.int32)
        if state_row.numel() < B:
            raise KernelError("state_row is smaller than the batch")
    elif R < B:
        raise KernelError(f"{R} sampler states for {B} rows")
    check_sampler(temperature, top_k, top_p, min_p, V)
    vpad = 0
    if needs_sort_scratch(temperature, top_k, top_p, min_p, V):
        vpad = sort_scratch_size(V)
        if sort_key is None:
            sort_key = empty((B, vpad), torch.float32, logits.device)
            sort_idx = empty((B, vpad), torch.int32, logits.device)
        _need(sort_key, "sort_key", torch.float32)
        _need(sort_idx, "sort_idx", torch.int32)
        if sort_key.numel() < B * vpad or sort_idx.numel() < B * vpad:
            raise KernelError("sorting scratch is smaller than the batch needs")
    a = _SampleArgs(logits.data_ptr(), work.data_ptr(), _addr(state_row), recent.data_ptr(),
                    recent_n.data_ptr(), rng.data_ptr(), out.data_ptr(), _addr(sort_key), _addr(sort_idx),
                    B, V, vpad, top_k,
                    temperature, top_p, min_p, repeat_penalty)
    _check(_launch(_lib("sampling.cu").gl_sample, byref(a), _stream()), "sample")


def set_pdl(on: bool) -> None:
    """Switch programmatic dependent launch on or off in every library loaded so far (on by
    default).  With it a kernel's blocks may be scheduled, and a product may start fetching
    its weights, while the kernel before it is still finishing."""
    for lib in list(build._loaded.values()):
        if hasattr(lib, "gl_set_pdl"):
            lib.gl_set_pdl(c_int(1 if on else 0))


def warm_up(head_dims=()) -> None:
    """Compile (if needed) and load every library a model with these head sizes uses."""
    for src, defines in catalog.all_libraries(head_dims):
        _lib(src, defines)
