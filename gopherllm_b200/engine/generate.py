"""The generation loop above the step function.

Requests (prompts of token ids) are cut into batches that fit the cache; the
prompts of a batch run in one step, then every live sequence gets one token per
step.  A sequence that ends leaves the batch at once and its slot and pages go
back to the cache; the next batch reuses them.  Per sequence the order of
events is the reference's (runtime.go:1130-1165, emitToken :1059-1095): sample
from the current logits; a stop token ends the sequence with "stop" and is
neither emitted nor fed; otherwise the token is emitted, and the sequence ends
with "length" once max_tokens are out or the cache cannot take another
position; otherwise the token is fed.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence, Tuple

from ..cache.sequence_cache import PAGE
from ..sampling.sampler import DeviceSampler, SamplerConfig, request_seed


@dataclass
class GenerationOptions:
    """The reference's GenerationOptions (runtime.go:90-125) for token-level use:
    max_tokens (default 256), sampler, seed (0: taken from the clock,
    runtime.go:906-910), stop_tokens (default: the model's end-of-sequence id,
    runtime.go:1914), should_stop (polled between steps, as the reference polls
    its context, runtime.go:1131), on_token(request index, token): called for every
    emitted token as it is known; returning False cancels the generation with what
    was generated so far (the reference's streaming callback, runtime.go:793-815,
    1024, which gets text; this library is token-level)."""
    max_tokens: int = 256
    sampler: SamplerConfig = field(default_factory=SamplerConfig)
    seed: int = 0
    stop_tokens: Tuple[int, ...] = ()
    should_stop: Optional[Callable[[], bool]] = None
    on_token: Optional[Callable[[int, int], Optional[bool]]] = None

    @classmethod
    def from_kwargs(cls, spec=None, **kw) -> "GenerationOptions":
        s = SamplerConfig()
        for k in ("temperature", "top_p", "top_k", "min_p", "repeat_penalty"):
            if k in kw:
                setattr(s, k, kw.pop(k))
        if "sampler" in kw:
            s = kw.pop("sampler")
        stops = kw.pop("stop_tokens", None)
        if stops is None:
            stops = tuple(spec.stop_tokens) if spec is not None else ()
        o = cls(max_tokens=kw.pop("max_tokens", 256), sampler=s, seed=kw.pop("seed", 0),
                stop_tokens=tuple(int(t) for t in stops), should_stop=kw.pop("should_stop", None),
                on_token=kw.pop("on_token", None))
        if kw:
            raise TypeError(f"unknown generation options: {', '.join(sorted(kw))}")
        return o

    def validate(self) -> None:
        if not isinstance(self.max_tokens, int) or self.max_tokens <= 0:
            raise ValueError("max_tokens must be greater than 0")
        self.sampler.validate()


@dataclass
class GenerationStats:
    """runtime.go:198-205; times in seconds."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    ttft: float = 0.0
    prefill_time: float = 0.0
    decode_time: float = 0.0
    total_time: float = 0.0
    token_times: List[float] = field(default_factory=list)   # seconds from the request's start to each token


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str          # "stop", "length" or "canceled"
    stats: GenerationStats


class GenerationCanceled(RuntimeError):
    """should_stop() returned true; ``results`` holds what was generated so far."""

    def __init__(self, results):
        super().__init__("generation canceled")
        self.results = results


# ---------------------------------------------------------------------------
# decisions (no device involved)
# ---------------------------------------------------------------------------
def pages_for(prompt_len: int, max_tokens: int, max_positions: int) -> int:
    """Pages a request can come to hold: its prompt plus every token it may feed."""
    return -(-min(prompt_len + max_tokens, max_positions) // PAGE)


def plan_batches(prompt_lens: Sequence[int], max_tokens: int, max_positions: int,
                 page_budget: int, slot_budget: int) -> List[List[int]]:
    """Cut requests, in order, into batches whose worst-case page need fits the cache."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, n in enumerate(prompt_lens):
        if n < 1:
            raise ValueError(f"request {i}: the prompt is empty")
        if n >= max_positions:
            # the reference rejects len(tokens) >= MaxSeqLen before any forward (runtime.go:866-868)
            raise ValueError(f"request {i}: prompt of {n} tokens does not fit {max_positions} positions")
        need = pages_for(n, max_tokens, max_positions)
        if need > page_budget:
            raise ValueError(f"request {i} needs {need * PAGE} cached positions, the cache holds {page_budget * PAGE}")
        if cur and (used + need > page_budget or len(cur) >= slot_budget):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class SequenceState:
    """One request's progress; ``accept`` is the per-token decision."""

    def __init__(self, prompt: Sequence[int], max_tokens: int, stop_tokens, max_positions: int):
        self.prompt = list(prompt)
        self.max_tokens, self.max_positions = max_tokens, max_positions
        self.stop_tokens = frozenset(int(t) for t in stop_tokens)
        self.generated: List[int] = []
        self.fed = len(self.prompt)          # positions in the cache
        self.finish_reason: Optional[str] = None

    def may_continue(self) -> bool:
        """Whether a next token that is no stop token would be fed for another step."""
        return len(self.generated) + 1 < self.max_tokens and self.fed < self.max_positions

    def accept(self, token: int) -> bool:
        """Take the sampled token; True if it must be fed for another step."""
        if self.finish_reason is not None:
            raise RuntimeError("sequence already finished")
        if token in self.stop_tokens:
            self.finish_reason = "stop"
            return False
        self.generated.append(int(token))
        if len(self.generated) >= self.max_tokens or self.fed >= self.max_positions:
            self.finish_reason = "length"
            return False
        self.fed += 1
        return True


# ---------------------------------------------------------------------------
def generate(engine, prompts: Sequence[Sequence[int]], options: GenerationOptions) -> List[GenerationResult]:
    options.validate()
    import torch
    spec = engine.model.spec
    cache = engine.cache
    seed = options.seed if options.seed != 0 else time.time_ns()
    batches = plan_batches([len(p) for p in prompts], options.max_tokens, spec.max_positions,
                           cache.n_pages, cache.max_slots)
    results: List[Optional[GenerationResult]] = [None] * len(prompts)
    prepare = getattr(engine, "prepare_decode", None)
    # kernels that gave up a bounded wait leave a status word: read where the host waits anyway, so that
    # an invalid result is an error here, as errors of the reference's forward pass end its loop
    # (runtime.go:1131-1165), and not a wrong token
    check = getattr(engine, "check_device", lambda: None)
    fetch = getattr(engine, "fetch", None) if prepare is not None else None
    for batch in batches:
        t_start = time.perf_counter()
        states = [SequenceState(prompts[i], options.max_tokens, options.stop_tokens, spec.max_positions)
                  for i in batch]
        sampler = DeviceSampler(options.sampler, [request_seed(seed, i) for i in batch],
                                [prompts[i] for i in batch], spec.vocab, engine.device)
        slots = [engine.open() for _ in batch]
        stats = [GenerationStats(prompt_tokens=len(prompts[i])) for i in batch]
        live = list(range(len(batch)))
        canceled = False
        try:
            logits = engine.step([(slots[r], states[r].prompt) for r in live])
            rows_dev = None
            first = True
            t_prefill_end = None
            while live:
                if rows_dev is None:
                    rows_dev = torch.tensor(live, dtype=torch.int32).to(engine.device)
                chosen = sampler.sample(logits, rows_dev)
                # While the device finishes the step and samples: the next step's descriptor, if every
                # sequence can go on.  An engine that can read its tokens on the device is given the
                # sampler's output and starts that step at once, before the host has seen the tokens, so
                # the device does not wait for the host between steps; should a sequence then end with
                # a stop token, the step has merely fed one token too many to a sequence that is closed,
                # and the rows of the others stand (a row does not depend on its neighbours).
                ahead, ahead_logits, sampled = None, None, None
                if prepare is not None and all(states[r].may_continue() for r in live):
                    ahead = prepare([slots[r] for r in live])
                    if fetch is not None:
                        sampled = torch.cuda.Event()
                        sampled.record()
                        ahead_logits = engine.finish_decode(ahead, chosen)
                        ahead = None
                tokens = fetch(chosen, sampled) if sampled is not None else chosen.tolist()   # waits for the sampling
                now = time.perf_counter()
                if first:
                    check()                      # the prompts' step is over: the host has its tokens
                    t_prefill_end = now
                    for r in live:
                        stats[r].prefill_time = now - t_start
                        stats[r].ttft = now - t_start
                    first = False
                nxt, runs, kept = [], [], []
                for i, (r, tok) in enumerate(zip(live, tokens)):
                    stats[r].token_times.append(now - t_start)
                    emitted = len(states[r].generated)
                    goes_on = states[r].accept(tok)
                    if options.on_token is not None and len(states[r].generated) > emitted:
                        if options.on_token(batch[r], tok) is False:
                            canceled = True
                    if goes_on:
                        nxt.append(r)
                        runs.append((slots[r], [tok]))
                        kept.append(i)
                    else:
                        engine.close(slots[r])
                        slots[r] = None
                        stats[r].total_time = now - t_start
                        stats[r].decode_time = now - t_prefill_end
                if len(nxt) != len(live):
                    rows_dev = None
                live = nxt
                if canceled or (options.should_stop is not None and options.should_stop()):
                    canceled = True
                    break
                if runs:
                    if ahead_logits is not None:
                        logits = ahead_logits if len(kept) == len(tokens) else \
                            ahead_logits.index_select(0, torch.tensor(kept, dtype=torch.int64).to(engine.device))
                    elif ahead is not None and len(runs) == len(tokens):
                        logits = engine.finish_decode(ahead, tokens)
                    else:
                        logits = engine.step(runs)
            check()                              # the batch is over and the host has waited for its last tokens
        finally:
            for s in slots:
                if s is not None:
                    engine.close(s)
        now = time.perf_counter()
        for r, i in enumerate(batch):
            st = states[r]
            if st.finish_reason is None:
                st.finish_reason = "canceled"
                stats[r].total_time = now - t_start
                stats[r].decode_time = now - (t_prefill_end or now)
            stats[r].generated_tokens = len(st.generated)
            results[i] = GenerationResult(st.generated, st.finish_reason, stats[r])
        if canceled:
            done = [r if r is not None else GenerationResult([], "canceled", GenerationStats()) for r in results]
            raise GenerationCanceled(done)
    return results
