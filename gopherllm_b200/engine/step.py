"""The step function: one batch of token runs through the model, from the cache.

A step takes, for each sequence of the batch, its next tokens (a whole prompt, a
piece of one, or a single token) and the places among them whose logits are
wanted.  It runs exactly those tokens as one ragged batch (no padding exists,
so padding cannot change a result), writes their keys and values behind what
the cache already holds for the sequence, and returns float32 logits at the
wanted places.  The reference has the two ends of this: a chunk of one sequence
(ForwardBatchInto, forward_batch.go:311-318, logits for the last position only,
:601-612) and a single token (ForwardInto, model.go:2550-2553).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.sequence_cache import PAGE, SequenceCache
from .model import DecoderModel


class StepContext:
    """What the parts see of a step.  Tensors are int32 on the device.

    tokens[T], tok_seq[T] (index of the token's sequence in this batch),
    tok_pos[T] (absolute position); seq_slot[B], seq_qstart[B] (row of the
    sequence's first token), seq_qlen[B], seq_ctx[B] (positions cached before
    the step); want_rows[M]; pages[g] = [B, max_pages] page ids in cache group g.
    Host-side: n_tokens, n_seqs, n_want, max_qlen, max_len (longest sequence
    after the step), is_decode (every run is one token), act_dtype, device,
    scratch (per-step memo shared by the parts, e.g. position tables).
    """

    def __init__(self, device, act_dtype):
        self.device, self.act_dtype = device, act_dtype
        self.scratch: Dict = {}
        self.pages: List[torch.Tensor] = []
        self.tokens = self.tok_seq = self.tok_pos = None
        self.seq_slot = self.seq_qstart = self.seq_qlen = self.seq_ctx = None
        self.want_rows = None
        self.n_tokens = self.n_seqs = self.n_want = 0
        self.max_qlen = self.max_len = 0
        self.is_decode = False
        self.side_stream = None          # a second stream blocks may fork onto (decode steps only)


def _pad4(n: int) -> int:
    return (n + 3) & ~3


class _Layout:
    """Offsets of the step's arrays inside one int32 buffer (each 16-byte aligned)."""

    def __init__(self, T: int, B: int, M: int, groups: int, max_pages: int):
        self.T, self.B, self.M, self.groups, self.max_pages = T, B, M, groups, max_pages
        o = 0
        self.off: Dict[str, Tuple[int, int]] = {}
        for name, n in (("tokens", T), ("tok_seq", T), ("tok_pos", T), ("seq_slot", B),
                        ("seq_qstart", B), ("seq_qlen", B), ("seq_ctx", B), ("want_rows", M)):
            self.off[name] = (o, n)
            o += _pad4(n)
        for g in range(groups):
            self.off[f"pages{g}"] = (o, B * max_pages)
            o += _pad4(B * max_pages)
        self.size = max(o, 4)

    def key(self):
        return (self.T, self.B, self.M, self.groups, self.max_pages)


class Engine:
    """Owns a model, its cache and the step function."""

    def __init__(self, model: DecoderModel, cache: SequenceCache, act_dtype: torch.dtype, device):
        self.model, self.cache = model, cache
        self.act_dtype, self.device = act_dtype, torch.device(device)
        self.vocab = model.spec.vocab
        # decode steps (one token per sequence) of the bfloat16 path replay a CUDA graph per
        # batch shape; the 32-bit path always launches kernel by kernel
        self.use_graphs = act_dtype == torch.bfloat16 and bool(getattr(model, "capturable", False))
        self.graph_max_batch = 256
        self.graph_first_runs = 2                            # runs of the schedule in a step's first, short graph
        self._graphs: Dict[tuple, object] = {}             # insertion order = least recently used first
        self.graph_limit = 64                                # captured steps kept (each holds its logits and descriptor)
        self._graph_pool = None
        self.overlap_branches = True                         # decode steps run parallel branches on two streams
        self._side_stream = None
        self._copy_stream = None
        self._fetch_pin = None
        self.launches_per_loop_step: Dict[int, int] = {}    # kernels in one captured decode_loop step, by batch
        self._pinned: List[Optional[torch.Tensor]] = [None, None]
        self._events: List[Optional[torch.cuda.Event]] = [None, None]
        self._flip = 0
        self.h2d_bytes_last = 0
        self._logits_aliased = False                         # the last launch returned a captured graph's buffer

    # -- sequences ----------------------------------------------------------
    def open(self) -> int:
        return self.cache.open()

    def close(self, slot: int) -> None:
        self.cache.close(slot)

    def check_device(self) -> None:
        """Raise KernelError if a kernel gave up a bounded wait since the last check (its results, and
        everything computed from them, are invalid).  Reading the status words synchronises with the
        device, so callers do it where they wait for the device anyway: after a step whose results they
        copy to the host, at the end of a batch."""
        from .. import ops
        ops.check_wait_failures()

    # -- the step -------------------------------------------------------------
    def plan(self, runs: Sequence[Tuple[int, Sequence[int]]], want: Optional[Sequence[Sequence[int]]]):
        """Host-side part of a step: checks, page reservation, the packed descriptor.
        Returns (layout, numpy int32 buffer, new lengths)."""
        if not runs:
            raise ValueError("a step needs at least one sequence")
        cache = self.cache
        slots = [int(s) for s, _ in runs]
        if len(set(slots)) != len(slots):
            raise ValueError("a sequence appears twice in one step")
        qlens = [len(t) for _, t in runs]
        if min(qlens) < 1:
            raise ValueError("every sequence of a step brings at least one token")
        ctxs = [cache.length(s) for s in slots]
        T, B = sum(qlens), len(runs)
        if want is None:
            want = [[q - 1] for q in qlens]
        if len(want) != B:
            raise ValueError("want must have one list per sequence")
        rows: List[int] = []
        start = 0
        for q, w in zip(qlens, want):
            for i in w:
                if not 0 <= int(i) < q:
                    raise ValueError(f"wanted place {i} is outside a run of {q} tokens")
                rows.append(start + int(i))
            start += q
        toks = np.concatenate([np.asarray(t, dtype=np.int64) for _, t in runs])
        if toks.min() < 0 or toks.max() >= self.vocab:
            raise ValueError(f"token id outside [0, {self.vocab})")
        # every check that can refuse the step comes before this line: a refused step holds nothing
        cache.reserve([(s, c + q) for s, c, q in zip(slots, ctxs, qlens)])
        lay = _Layout(T, B, len(rows), len(cache.groups), cache.max_pages_per_seq)
        buf = np.zeros(lay.size, dtype=np.int32)

        def put(name, values):
            o, n = lay.off[name]
            buf[o:o + n] = values

        put("tokens", toks)
        put("tok_seq", np.repeat(np.arange(B), qlens))
        put("tok_pos", np.concatenate([np.arange(c, c + q) for c, q in zip(ctxs, qlens)]))
        put("seq_slot", slots)
        put("seq_qstart", np.concatenate([[0], np.cumsum(qlens)[:-1]]))
        put("seq_qlen", qlens)
        put("seq_ctx", ctxs)
        put("want_rows", rows)
        for g in range(lay.groups):
            o, n = lay.off[f"pages{g}"]
            cache.page_rows(g, slots, out=buf[o:o + n].reshape(B, lay.max_pages))
        meta = dict(slots=slots, new_lens=[c + q for c, q in zip(ctxs, qlens)],
                    max_qlen=max(qlens), is_decode=max(qlens) == 1)
        return lay, buf, meta

    def _stage(self, buf: np.ndarray) -> torch.Tensor:
        """The descriptor in pinned host memory, ready for an asynchronous copy."""
        i = self._flip
        self._flip ^= 1
        if self._events[i] is not None:
            self._events[i].synchronize()          # the copy that last used this staging buffer is done
        pin = self._pinned[i]
        if pin is None or pin.numel() < buf.size:
            pin = torch.empty(max(buf.size, 4096), dtype=torch.int32, pin_memory=True)
            self._pinned[i] = pin
        pin[:buf.size].numpy()[...] = buf
        self._staged = i
        self.h2d_bytes_last = buf.size * 4
        return pin[:buf.size]

    def _staged_done(self) -> None:
        ev = torch.cuda.Event()
        ev.record()
        self._events[self._staged] = ev

    def context(self, lay: _Layout, dev: torch.Tensor, meta: dict) -> StepContext:
        ctx = StepContext(self.device, self.act_dtype)
        for name in ("tokens", "tok_seq", "tok_pos", "seq_slot", "seq_qstart", "seq_qlen",
                     "seq_ctx", "want_rows"):
            o, n = lay.off[name]
            setattr(ctx, name, dev[o:o + n])
        for g in range(lay.groups):
            o, n = lay.off[f"pages{g}"]
            ctx.pages.append(dev[o:o + n].view(lay.B, lay.max_pages))
        ctx.n_tokens, ctx.n_seqs, ctx.n_want = lay.T, lay.B, lay.M
        ctx.max_qlen, ctx.is_decode = meta["max_qlen"], meta["is_decode"]
        ctx.max_len = max(meta["new_lens"])
        if ctx.is_decode and self.overlap_branches and self.act_dtype == torch.bfloat16:
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=self.device)
            ctx.side_stream = self._side_stream
        return ctx

    @torch.no_grad()
    def step(self, runs: Sequence[Tuple[int, Sequence[int]]],
             want: Optional[Sequence[Sequence[int]]] = None) -> torch.Tensor:
        """runs: [(slot, tokens)]; want[b]: places in run b whose logits are wanted
        (default: the last token of every run).  Returns float32 [wanted, vocab] on
        the device, in the order of runs and of want."""
        lay, buf, meta = self.plan(runs, want)
        logits = self._launch(lay, self._stage(buf), meta)
        # a replayed step leaves its logits in the captured graph's own buffer, which the next step of
        # the same shape overwrites: the caller gets a tensor that stays as it is
        return logits.clone() if self._logits_aliased else logits

    def prepare_decode(self, slots: Sequence[int]):
        """The host's share of a one-token step that does not depend on the tokens themselves:
        page reservation, positions, page tables, the staged descriptor.  A generation loop calls
        this while the device still works on the step before, then ``finish_decode`` with the
        sampled tokens; a handle that is not finished (the batch changed) is simply dropped."""
        lay, buf, meta = self.plan([(s, (0,)) for s in slots], None)
        return lay, self._stage(buf), meta

    def finish_decode(self, handle, tokens) -> torch.Tensor:
        """Launch a prepared one-token step.  ``tokens``: one id per sequence from the host, or an
        int32 tensor on the device (a sampler's output): the step then reads its tokens where the
        sampler left them, so it can be launched before the host has seen them.  The logits of a
        replayed step are the captured graph's own buffer: they hold until the next step of the same
        shape (``step`` hands out a copy instead)."""
        lay, pin, meta = handle
        o, n = lay.off["tokens"]
        if isinstance(tokens, torch.Tensor):
            if tokens.dtype != torch.int32 or tokens.shape != (n,) or tokens.device != self.device:
                raise ValueError(f"{n} int32 tokens on {self.device} expected, one per sequence")
            return self._launch(lay, pin, meta, tokens_dev=tokens)
        toks = np.asarray(tokens, dtype=np.int64)
        if toks.shape != (n,):
            raise ValueError(f"{n} tokens expected, one per sequence")
        if toks.min() < 0 or toks.max() >= self.vocab:
            raise ValueError(f"token id outside [0, {self.vocab})")
        pin.numpy()[o:o + n] = toks
        return self._launch(lay, pin, meta)

    def fetch(self, values: torch.Tensor, after: "torch.cuda.Event") -> List[int]:
        """A small device tensor as a host list, copied on a stream of its own once ``after`` has
        happened: work queued behind ``after`` on the main stream does not hold the copy up."""
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream(device=self.device)
        n = values.numel()
        if self._fetch_pin is None or self._fetch_pin.numel() < n or self._fetch_pin.dtype != values.dtype:
            self._fetch_pin = torch.empty(max(n, 1024), dtype=values.dtype, pin_memory=True)
        s = self._copy_stream
        s.wait_event(after)
        with torch.cuda.stream(s):
            self._fetch_pin[:n].copy_(values.reshape(-1), non_blocking=True)
            done = torch.cuda.Event()
            done.record(s)
        done.synchronize()
        return self._fetch_pin[:n].tolist()

    def _launch(self, lay: _Layout, pin: torch.Tensor, meta: dict,
                tokens_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
        graph = None
        self._logits_aliased = False
        if self.use_graphs and meta["is_decode"] and lay.B <= self.graph_max_batch:
            graph = self._decode_graph(lay, meta)
        o, n = lay.off["tokens"]
        if graph is not None:
            graph.desc.copy_(pin, non_blocking=True)
            if tokens_dev is not None:
                graph.desc[o:o + n].copy_(tokens_dev)
            self._staged_done()
            graph.first.replay()
            if graph.graph is not None:
                graph.graph.replay()
            logits = graph.logits
            self._logits_aliased = True
        else:
            dev = torch.empty(lay.size, dtype=torch.int32, device=self.device)
            dev.copy_(pin, non_blocking=True)
            if tokens_dev is not None:
                dev[o:o + n].copy_(tokens_dev)
            self._staged_done()
            logits = self.model.forward(self.context(lay, dev, meta), self.cache)
        for s, n in zip(meta["slots"], meta["new_lens"]):
            self.cache.commit(s, n)
        return logits

    # -- CUDA graphs for decode steps -------------------------------------------
    def _length_bucket(self, longest: int) -> int:
        """Sequence lengths share a captured step by bucket (4, 8, 16, ... pages, at most the cache's
        longest sequence): how a kernel cuts its work may depend on the length (the splits of decode
        attention), never whether its result is right, so a bucket's graph is sized for its upper end."""
        pages = 4
        while pages * PAGE < longest:
            pages *= 2
        return min(pages * PAGE, self.cache.max_positions)

    def _decode_graph(self, lay: _Layout, meta: dict):
        """The captured step for this batch shape, or None the first time the shape is
        seen (that step runs kernel by kernel, which also loads and warms every kernel).
        The logits of a replayed step live in the graph's own buffer until the next
        replay of the same shape."""
        bucket = self._length_bucket(max(meta["new_lens"]))
        key = lay.key() + (bucket,)
        g = self._graph_lookup(key)
        if g is None:
            self._graph_store(key, False)
            return None
        if g is False:
            g = _CapturedStep()
            g.desc = torch.zeros(lay.size, dtype=torch.int32, device=self.device)
            bound = dict(meta)
            bound["new_lens"] = [bucket]                        # launch sizes are chosen for the bucket's longest
            ctx = g.ctx = self.context(lay, g.desc, bound)     # lives as long as the graphs: they read its tables
            torch.cuda.synchronize(self.device)
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            # Two graphs replayed back to back: a short one (the embedding and the first runs of the
            # schedule) that the device can start soon after the launch call, and the rest, whose
            # longer launch is then hidden behind the first one's work.  A step that is launched from
            # an idle device (the generation loop waits for each step's tokens) otherwise pays the
            # whole launch of a few hundred nodes before its first kernel.
            n_runs = len(self.model.spec.schedule)
            n_first = min(self.graph_first_runs, n_runs)
            g.first = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g.first, pool=self._graph_pool):
                g.x = self.model.begin(ctx)
                self.model.run(g.x, ctx, self.cache, 0, n_first)
                if n_first == n_runs:
                    g.logits = self.model.finish(g.x, ctx)
            g.graph = None
            if n_first < n_runs:
                g.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g.graph, pool=self._graph_pool):
                    self.model.run(g.x, ctx, self.cache, n_first, n_runs)
                    g.logits = self.model.finish(g.x, ctx)
            self._graph_store(key, g)
        return g

    def _graph_lookup(self, key):
        g = self._graphs.get(key)
        if g is not None:
            self._graphs[key] = self._graphs.pop(key)        # most recently used last
        return g

    def _graph_store(self, key, g) -> None:
        self._graphs.pop(key, None)
        self._graphs[key] = g
        while len(self._graphs) > self.graph_limit:          # the least recently used shape goes
            del self._graphs[next(iter(self._graphs))]

    @torch.no_grad()
    def decode_loop(self, slots: Sequence[int], tokens: Sequence[int], steps: int, sampler) -> torch.Tensor:
        """Run ``steps`` decode steps for these sequences wholly on the device: each step
        feeds the tokens the sampler chose in the step before (the first step feeds
        ``tokens``).  Pages for all steps are reserved first.  Returns the chosen tokens,
        int32 [steps, len(slots)], on the device; nothing is copied to the host in between."""
        from .. import ops
        if steps < 1:
            raise ValueError("steps must be at least 1")
        history_cap = 4096
        if steps > history_cap:
            raise ValueError(f"decode_loop runs at most {history_cap} steps a call")
        cache = self.cache
        B = len(slots)
        if len(tokens) != B or len(set(int(s) for s in slots)) != B:
            raise ValueError("decode_loop takes one token for each of its distinct sequences")
        if min(int(t) for t in tokens) < 0 or max(int(t) for t in tokens) >= self.vocab:
            raise ValueError(f"token id outside [0, {self.vocab})")
        ctxs = [cache.length(s) for s in slots]
        # pages for all steps first: the page table staged below then covers every position of the loop
        cache.reserve([(s, c + steps) for s, c in zip(slots, ctxs)])
        lay, buf, meta = self.plan([(s, [t]) for s, t in zip(slots, tokens)], None)
        pin = self._stage(buf)
        bucket = self._length_bucket(max(ctxs) + steps)
        # a captured loop step has its sampler's options and state buffers as kernel arguments
        key = ("loop", id(sampler)) + lay.key() + (bucket,)
        g = self._graph_lookup(key)
        if g is None:
            g = _CapturedStep()
            g.desc = torch.zeros(lay.size, dtype=torch.int32, device=self.device)
            g.counter = torch.zeros(1, dtype=torch.int32, device=self.device)
            g.history = torch.zeros((history_cap, B), dtype=torch.int32, device=self.device)
            g.state_row = torch.arange(B, dtype=torch.int32, device=self.device)
            g.sampler = sampler
            g.bound = dict(meta)
            g.bound["new_lens"] = [bucket]                     # launch sizes are chosen for the bucket's longest

        def body(ctx):
            logits = self.model.forward(ctx, cache)
            chosen = g.sampler.sample(logits, g.state_row)
            ops.advance_decode(ctx.tokens, ctx.tok_pos, ctx.seq_ctx, chosen, g.history, g.counter)

        if g.graph is None and getattr(self.model, "capturable", False):
            g.desc.copy_(pin, non_blocking=True)
            # Once kernel by kernel, which loads and warms everything, with a context of its own: what
            # the parts memoise per step (position tables) must be computed again inside the capture,
            # or the graph would go on reading the warm-up step's tables at every position.  The
            # warm-up leaves no trace: the sampler's state and the sequences' state rows are put back,
            # and the keys and values it wrote are written again, equal, by the first replay.
            saved = [t.clone() for t in (sampler.rng, sampler.recent, sampler.recent_n)]
            states = cache.state_snapshot(slots)
            body(self.context(lay, g.desc, g.bound))
            for t, keep in zip((sampler.rng, sampler.recent, sampler.recent_n), saved):
                t.copy_(keep)
            cache.state_restore(slots, states)
            torch.cuda.synchronize(self.device)
            g.ctx = self.context(lay, g.desc, g.bound)        # fresh, and kept with the graph that reads its tables
            g.graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            before = ops.LAUNCHES
            with torch.cuda.graph(g.graph, pool=self._graph_pool):
                body(g.ctx)
            self.launches_per_loop_step[B] = ops.LAUNCHES - before
        self._graph_store(key, g)
        g.desc.copy_(pin, non_blocking=True)
        self._staged_done()
        g.counter.zero_()
        if g.graph is not None:
            for _ in range(steps):
                g.graph.replay()
        else:                                                   # a model with a part that cannot be captured
            for _ in range(steps):
                body(self.context(lay, g.desc, g.bound))
        for s, c in zip(slots, ctxs):
            cache.commit(s, c + steps)
        return g.history[:steps]


class _CapturedStep:
    """A CUDA graph of one step with the buffers it reads and writes, and the step context it was
    captured with (whose per-step memos, such as position tables, are nodes' outputs in the graph)."""
    desc = graph = logits = ctx = bound = None
