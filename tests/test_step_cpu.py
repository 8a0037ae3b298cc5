"""The step function's host side and the failure checks, without a device."""
import numpy as np
import pytest
import torch

from gopherllm_b200.cache.sequence_cache import SequenceCache
from gopherllm_b200.engine.generate import GenerationOptions, generate
from gopherllm_b200.engine.step import Engine
from gopherllm_b200.parts.base import KVRequest
from gopherllm_b200.sampling.sampler import SamplerConfig


class _Spec:
    vocab = 100
    max_positions = 256
    stop_tokens = ()


class _Net:
    spec = _Spec()
    capturable = False


def engine(max_tokens=512):
    cache = SequenceCache([KVRequest(2, 16), KVRequest(2, 16)], max_tokens, 256, torch.float32, "cpu", allocate=False)
    return Engine(_Net(), cache, torch.float32, "cpu")


def test_a_refused_step_holds_nothing():
    """Token ids and wanted places are checked before pages are reserved: a step that is refused
    leaves the sequences' pages and lengths as they were."""
    eng = engine()
    cache = eng.cache
    a, b = eng.open(), eng.open()
    cache.reserve([(a, 10)])
    cache.commit(a, 10)
    held = cache.groups[0].pool.held_count
    for runs, want in (([(a, [1, 2, 100])], None),               # id == vocabulary
                       ([(a, [1]), (b, [-1] * 70)], None),       # negative id, in a run that would need two pages
                       ([(a, list(range(80)))], [[80]]),         # wanted place outside the run
                       ([(a, [1]), (a, [2])], None),             # a sequence twice
                       ([(a, [])], None)):
        with pytest.raises(ValueError):
            eng.plan(runs, want)
        assert cache.groups[0].pool.held_count == held and cache.length(a) == 10 and cache.length(b) == 0
        assert cache.pages_needed(b, 64) == 1
        cache.check()
    lay, buf, meta = eng.plan([(a, [5, 6]), (b, list(range(70)))], [[1], [0, 69]])
    assert cache.groups[0].pool.held_count == held + 2 and meta["new_lens"] == [12, 70]
    o, n = lay.off["want_rows"]
    assert list(buf[o:o + n]) == [1, 2, 71]
    o, n = lay.off["tok_pos"]
    assert list(buf[o:o + 3]) == [10, 11, 0]
    with pytest.raises(ValueError):
        eng.decode_loop([a, b], [1, 100], 3, None)               # a bad id reserves nothing either
    assert cache.groups[0].pool.held_count == held + 2
    cache.check()


def test_a_wait_that_ran_out_is_an_error_not_a_wrong_result(monkeypatch):
    from gopherllm_b200 import ops
    words = {"libgl_gemm_skinny": 0, "libgl_gemm_tcgen05": 1, "libgl_attention_prefill_tc_head_dim80": -1}
    cleared = []

    def fake(clear=False):
        out = dict(words)
        if clear:
            cleared.append(True)
            for k in words:
                words[k] = 0
        return out
    monkeypatch.setattr(ops, "wait_failures", fake)
    with pytest.raises(ops.KernelError) as e:
        engine().check_device()
    assert "libgl_gemm_tcgen05" in str(e.value) and "libgl_attention_prefill_tc_head_dim80" in str(e.value)
    assert "libgl_gemm_skinny" not in str(e.value) and cleared
    engine().check_device()                                      # cleared: the next check speaks of what ran since


class _FakeEngine:
    """Just enough of an engine for the generation loop: logits that always choose token 5."""
    device = "cpu"

    def __init__(self, fail_at):
        self.model = _Net()
        self.cache = SequenceCache([KVRequest(1, 16)], 1024, 256, torch.float32, "cpu", allocate=False)
        self.checks, self.fail_at, self.closed = 0, fail_at, 0

    def open(self):
        return self.cache.open()

    def close(self, s):
        self.closed += 1
        self.cache.close(s)

    def step(self, runs, want=None):
        self.cache.reserve([(s, self.cache.length(s) + len(t)) for s, t in runs])
        for s, t in runs:
            self.cache.commit(s, self.cache.length(s) + len(t))
        out = torch.zeros((len(runs), 100))
        out[:, 5] = 1.0
        return out

    def check_device(self):
        from gopherllm_b200.ops import KernelError
        self.checks += 1
        if self.checks == self.fail_at:
            raise KernelError("a kernel gave up waiting")


def test_generate_reads_the_failure_word_after_the_prompts_and_at_the_end(monkeypatch):
    from gopherllm_b200.engine import generate as gen
    from gopherllm_b200.ops import KernelError

    class HostSampler:
        def __init__(self, *a, **k):
            pass

        def sample(self, logits, rows=None):
            return logits.argmax(-1).to(torch.int32)
    monkeypatch.setattr(gen, "DeviceSampler", HostSampler)
    opts = GenerationOptions(max_tokens=4, sampler=SamplerConfig.greedy(), seed=1)
    ok = _FakeEngine(fail_at=0)
    res = generate(ok, [[1, 2, 3], [4]], opts)
    assert [r.tokens for r in res] == [[5] * 4, [5] * 4] and ok.checks == 2
    for fail_at in (1, 2):
        bad = _FakeEngine(fail_at)
        with pytest.raises(KernelError):
            generate(bad, [[1, 2, 3], [4]], opts)
        assert bad.cache.slots.held_count == 0          # the batch's slots went back all the same
        bad.cache.check()
