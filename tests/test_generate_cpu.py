"""The generation loop's decisions and the options' rules (no device needed)."""
import pytest

from gopherllm_b200.engine.generate import GenerationOptions, SequenceState, pages_for, plan_batches
from gopherllm_b200.sampling.sampler import PRESETS, SamplerConfig, recent_window, request_seed
from gopherllm_b200.cli import build_parser, effective_sampler, parse_duration, parse_prompts


def test_accept_order_stop_emit_length_feed():
    # runtime.go:1130-1165: a stop token is neither emitted nor fed
    s = SequenceState([1, 2, 3], max_tokens=3, stop_tokens=[9], max_positions=100)
    assert s.accept(5) and s.generated == [5] and s.fed == 4
    assert not s.accept(9) and s.finish_reason == "stop" and s.generated == [5] and s.fed == 4
    with pytest.raises(RuntimeError):
        s.accept(1)
    s = SequenceState([1, 2, 3], max_tokens=2, stop_tokens=[], max_positions=100)
    assert s.accept(5)
    assert not s.accept(6) and s.finish_reason == "length" and s.generated == [5, 6] and s.fed == 4
    # the cache cannot take another position: the token is emitted, not fed
    s = SequenceState([1, 2, 3], max_tokens=50, stop_tokens=[], max_positions=4)
    assert s.accept(5) and s.fed == 4
    assert not s.accept(6) and s.finish_reason == "length" and s.generated == [5, 6]


def test_may_continue_foretells_accept():
    # the loop prepares the next step ahead only if every sequence would feed a token that is no stop token
    for max_tokens in (1, 2, 3, 7):
        for max_positions in (4, 5, 6, 50):
            s = SequenceState([1, 2, 3], max_tokens=max_tokens, stop_tokens=[9], max_positions=max_positions)
            while s.finish_reason is None:
                told = s.may_continue()
                assert s.accept(5) == told, (max_tokens, max_positions, s.generated)
    s = SequenceState([1, 2, 3], max_tokens=5, stop_tokens=[9], max_positions=50)
    assert s.may_continue() and not s.accept(9)           # a stop token ends it whatever was foretold


def test_plan_batches():
    P = 64
    # worst-case pages: prompt + every token it may feed, capped by the longest sequence
    assert pages_for(10, 20, 2048) == 1 and pages_for(60, 5, 2048) == 2 and pages_for(2000, 500, 2048) == 32
    assert plan_batches([10, 10, 10], 20, 2048, page_budget=2, slot_budget=8) == [[0, 1], [2]]
    assert plan_batches([10] * 5, 20, 2048, page_budget=100, slot_budget=2) == [[0, 1], [2, 3], [4]]
    assert plan_batches([100, 10, 300], 28, 2048, page_budget=6, slot_budget=8) == [[0, 1], [2]]
    with pytest.raises(ValueError, match="empty"):
        plan_batches([3, 0], 5, 64, 10, 10)
    with pytest.raises(ValueError, match="does not fit"):
        plan_batches([64], 5, 64, 10, 10)                 # len(tokens) >= MaxSeqLen (runtime.go:866-868)
    with pytest.raises(ValueError, match="the cache holds"):
        plan_batches([500], 500, 2048, page_budget=4, slot_budget=1)


def test_option_rules():
    GenerationOptions().validate()
    with pytest.raises(ValueError, match="max_tokens"):
        GenerationOptions(max_tokens=0).validate()
    bad = [dict(temperature=-1), dict(temperature=float("nan")), dict(top_p=0), dict(top_p=1.5),
           dict(top_k=-1), dict(min_p=2), dict(repeat_penalty=0)]
    for kw in bad:
        with pytest.raises(ValueError):
            GenerationOptions(sampler=SamplerConfig(**kw)).validate()
    d = SamplerConfig()
    assert (d.temperature, d.top_p, d.top_k, d.min_p, d.repeat_penalty) == (0.7, 0.9, 40, 0.0, 1.1)
    assert PRESETS["deterministic"].is_greedy and PRESETS["creative"].top_k == 80
    o = GenerationOptions.from_kwargs(None, max_tokens=5, temperature=0.0, stop_tokens=[1, 2], seed=7)
    assert o.max_tokens == 5 and o.sampler.is_greedy and o.stop_tokens == (1, 2) and o.seed == 7
    with pytest.raises(TypeError):
        GenerationOptions.from_kwargs(None, max_new_tokens=5)


def test_seeds_and_window():
    assert request_seed(5, 0) == 5 and request_seed(5, 3) == 8
    assert request_seed(0, 0) == 0xDEADBEEFCAFE1337          # zero is remapped (sampling.go:30-35)
    assert request_seed(2 ** 64 - 1, 1) == 0xDEADBEEFCAFE1337
    assert recent_window(list(range(100))) == list(range(36, 100)) and recent_window([1, 2]) == [1, 2]


def test_cli_options():
    assert parse_prompts("1, 2 3;4") == [[1, 2, 3], [4]]
    assert parse_duration("2m") == 120 and parse_duration("1h30m") == 5400 and parse_duration("500ms") == 0.5
    assert parse_duration("7") == 7.0
    with pytest.raises(SystemExit):
        parse_duration("soon")
    a = build_parser().parse_args(["m", "--preset", "precise", "--temp", "0.5", "-n", "7", "--top-k", "3"])
    s = effective_sampler(a)
    assert (s.temperature, s.top_k, s.top_p, s.repeat_penalty) == (0.5, 3, 0.9, 1.05) and a.max_tokens == 7
    a = build_parser().parse_args(["m"])
    assert effective_sampler(a) == SamplerConfig() and a.max_tokens is None and a.bench_runs == 3


def test_options_file(tmp_path, capsys):
    """--config: defaults, then the file's preset, the file's values, --preset, the other flags
    (cmd/gopherllm/main.go:686-707); unknown keys and versions are refused, the reference's keys that
    this library has no use for are read past."""
    import json
    from gopherllm_b200.cli import main
    f = tmp_path / "options.json"
    f.write_text(json.dumps({"version": 1, "preset": "precise", "model": "some/folder",
                             "generation": {"max_tokens": 33, "temperature": 0.4, "seed": 9, "stop": ["7", "8"],
                                            "system_prompt": "unused here"},
                             "runtime": {"timeout": "2m", "threads": 4}, "server": {"address": ":1"}}))

    def shown(*argv):
        assert main(list(argv) + ["--print-config"]) == 0
        return json.loads(capsys.readouterr().out)
    c = shown("--config", str(f))
    assert c["model"] == "some/folder" and c["max_tokens"] == 33 and c["seed"] == 9 and c["stop"] == ["7", "8"]
    assert c["timeout"] == "2m" and c["preset"] == "precise"
    assert c["sampler"] == dict(temperature=0.4, top_p=0.9, top_k=30, min_p=0.0, repeat_penalty=1.05)
    c = shown("other", "--config", str(f), "-n", "5", "--top-k", "2", "--seed", "4")      # flags win over the file
    assert c["model"] == "other" and c["max_tokens"] == 5 and c["seed"] == 4 and c["sampler"]["top_k"] == 2
    assert c["sampler"]["temperature"] == 0.4
    c = shown("--config", str(f), "--preset", "creative")                               # --preset resets the sampler
    assert c["sampler"] == dict(temperature=0.95, top_p=0.95, top_k=80, min_p=0.05, repeat_penalty=1.05)
    for bad in ({"version": 2}, {"generation": {"tempo": 1}}, {"colour": "red"}, {"preset": "wild"},
                {"runtime": {"timeout": "never"}}, [1, 2]):
        f.write_text(json.dumps(bad))
        with pytest.raises(SystemExit):
            main(["m", "--config", str(f), "--print-config"])
    with pytest.raises(SystemExit):
        main(["--print-config"])                                                        # no model anywhere


def test_decode_attention_splits_stay_within_the_machine():
    """How decode attention is cut over blocks is a launch decision made on the host: never more blocks
    than are resident at once, never more splits than pages or than a cluster holds, at least one."""
    from unittest import mock
    from gopherllm_b200 import ops
    with mock.patch.object(ops, "sm_count", lambda device: 148):
        for heads, hd in ((32, 80), (8, 128), (5, 32), (1, 256)):
            slots = 148 * ops.decode_blocks_per_sm(hd, 1)
            for batch in (1, 2, 3, 4, 7, 8, 16, 64, 300):
                last = 0
                for length in (1, 64, 65, 500, 1024, 2048, 8192, 100000):
                    s = ops.decode_splits(batch, heads, length, "cuda:0", hd, 1)
                    pages = -(-length // 64)
                    assert 1 <= s <= min(8, pages)
                    assert s == 1 or batch * heads * s <= slots
                    assert s >= last                      # a longer sequence is never cut into fewer parts
                    last = s
        # Phi-2 shapes: the measured best cuts
        assert [ops.decode_splits(b, 32, 2048, "cuda:0", 80, 1) for b in (1, 2, 4, 8, 16)] == [8, 4, 4, 2, 1]
        assert [ops.decode_splits(b, 32, 512, "cuda:0", 80, 1) for b in (2, 4, 8)] == [4, 2, 1]
