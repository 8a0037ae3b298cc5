"""Command line in the manner of the reference's ``gopherllm`` (cmd/gopherllm/main.go:26-103).

    python -m gopherllm_b200 MODEL_DIR --prompt "5 17 3" --max-tokens 32 --temp 0
    python -m gopherllm_b200 MODEL_DIR --bench-json --bench-runs 3
    python -m gopherllm_b200 MODEL_DIR --kernel-bench
    python -m gopherllm_b200 MODEL_DIR --inspect --list-tensors
    python -m gopherllm_b200 NEW_DIR --random-config config.json --seed 2

Options keep the reference's names and meanings where it has them (--prompt,
--max-tokens, --temp, --top-p, --top-k, --min-p, --repeat-penalty, --seed,
--preset, --stop, --bench, --bench-json, --bench-output, --bench-runs,
--kernel-bench, --kernel-bench-json, --kernel-bench-runs, --kernel-bench-layer,
--timeout, --inspect, --list-metadata, --list-tensors, --print-config).  A
prompt is a list of token ids (the library has no tokenizer): numbers separated
by spaces or commas; several prompts are separated by ";".
"""
from __future__ import annotations

import argparse
import json
import re
import sys
import time
from typing import List

from .sampling.sampler import PRESETS, SamplerConfig


def parse_prompts(text: str) -> List[List[int]]:
    prompts = []
    for part in text.split(";"):
        ids = [int(t) for t in re.split(r"[,\s]+", part.strip()) if t]
        if ids:
            prompts.append(ids)
    if not prompts:
        raise SystemExit("--prompt holds no token ids")
    return prompts


def parse_duration(text: str) -> float:
    """Go-style durations: 90s, 2m, 1h30m, 500ms; a bare number is seconds."""
    if re.fullmatch(r"[0-9.]+", text):
        return float(text)
    units = {"ms": 1e-3, "s": 1.0, "m": 60.0, "h": 3600.0}
    total, pos = 0.0, 0
    for m in re.finditer(r"([0-9.]+)(ms|s|m|h)", text):
        if m.start() != pos:
            break
        total += float(m.group(1)) * units[m.group(2)]
        pos = m.end()
    if pos != len(text) or pos == 0:
        raise SystemExit(f"--timeout {text!r} is not a duration such as 90s or 2m")
    return total


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="gopherllm_b200", description="Phi on one B200: generate, bench, inspect.")
    ap.add_argument("model", nargs="?", default=None,
                    help="model folder (config.json + model.safetensors); may come from --config instead")
    ap.add_argument("--config", dest="config_file", help="JSON file of options (version, preset, model, generation, runtime)")
    ap.add_argument("--prompt", "-p", help='token ids, e.g. "5 17 3"; ";" separates several prompts')
    ap.add_argument("--prompt-file", help="file with token ids, one prompt per line")
    ap.add_argument("--max-tokens", "-n", type=int, default=None, help="max tokens to generate (default: 256)")
    ap.add_argument("--temp", "-t", type=float, default=None, help="temperature (default: 0.7, 0=greedy)")
    ap.add_argument("--top-p", type=float, default=None, help="nucleus sampling threshold (default: 0.9)")
    ap.add_argument("--top-k", type=int, default=None, help="top-K filtering (default: 40)")
    ap.add_argument("--min-p", type=float, default=None, help="min-P sampling threshold (default: 0, disabled)")
    ap.add_argument("--repeat-penalty", type=float, default=None, help="repetition penalty (default: 1.1)")
    ap.add_argument("--seed", type=int, default=None, help="RNG seed (default: time-based)")
    ap.add_argument("--preset", choices=sorted(PRESETS), help="generation preset")
    ap.add_argument("--stop", action="append", default=None,
                    help="stop when this token id is sampled (repeatable; default: the model's eos_token_id)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--cache-tokens", type=int, default=None, help="positions the cache holds (default: 8 full sequences)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--bench", action="store_true", help="run a generation benchmark")
    ap.add_argument("--bench-json", action="store_true", help="run benchmark and emit machine-readable JSON")
    ap.add_argument("--bench-output", action="store_true", help="include generated tokens for each benchmark run")
    ap.add_argument("--bench-runs", type=int, default=3, help="number of benchmark runs (default: 3)")
    ap.add_argument("--kernel-bench", action="store_true", help="run isolated kernel benchmark")
    ap.add_argument("--kernel-bench-json", action="store_true", help="emit isolated kernel benchmark JSON")
    ap.add_argument("--kernel-bench-runs", type=int, default=25, help="number of kernel benchmark runs (default: 25)")
    ap.add_argument("--kernel-bench-layer", type=int, default=0, help="layer to benchmark (default: 0)")
    ap.add_argument("--timeout", default=None, help="abort generation or each benchmark run after a duration, e.g. 2m")
    ap.add_argument("--inspect", action="store_true", help="inspect config and tensors without loading weights")
    ap.add_argument("--list-metadata", action="store_true", help="print config.json keys with --inspect")
    ap.add_argument("--list-tensors", action="store_true", help="print the tensor inventory and exit")
    ap.add_argument("--print-config", action="store_true", help="print the effective options as JSON and exit")
    ap.add_argument("--random-config", help="write a random-weights model folder from this config.json, then exit")
    ap.add_argument("--verbose", "-v", action="store_true", help="log loading to stderr")
    return ap


CONFIG_VERSION = 1
# keys of the reference's options file (cmd/gopherllm/config.go:25-78); the ones this library has a use for
_FILE_KEYS = {"version", "preset", "model", "generation", "runtime"}
_FILE_GENERATION = {"max_tokens", "temperature", "top_p", "top_k", "min_p", "repeat_penalty", "seed", "stop"}
_FILE_RUNTIME = {"timeout"}
# and the ones it reads past (servers, model downloads, chat templates, CPU and Metal switches)
_FILE_IGNORED = {"model_dir", "server", "huggingface"}
_FILE_GENERATION_IGNORED = {"mtp_draft_tokens", "system_prompt", "context_window_mode"}
_FILE_RUNTIME_IGNORED = {"threads", "metal", "prepare_quant", "out_of_core", "auto_tune", "auto_refresh", "auto_effort"}


def load_file_config(path: str) -> dict:
    """The options file of --config: one JSON object, unknown keys refused, version 0 or 1
    (loadFileConfig, cmd/gopherllm/config.go:154-184)."""
    try:
        with open(path, "r", encoding="utf-8") as f:
            raw = json.load(f)
    except OSError as e:
        raise SystemExit(f"open config {path}: {e}")
    except json.JSONDecodeError as e:
        raise SystemExit(f"decode config {path}: {e}")
    if not isinstance(raw, dict):
        raise SystemExit(f"decode config {path}: expected one JSON object")

    def known(obj, allowed, ignored, where):
        if not isinstance(obj, dict):
            raise SystemExit(f"decode config {path}: {where} must be an object")
        extra = sorted(set(obj) - allowed - ignored)
        if extra:
            raise SystemExit(f"decode config {path}: unknown field {where + '.' if where else ''}{extra[0]}")
    known(raw, _FILE_KEYS, _FILE_IGNORED, "")
    known(raw.get("generation") or {}, _FILE_GENERATION, _FILE_GENERATION_IGNORED, "generation")
    known(raw.get("runtime") or {}, _FILE_RUNTIME, _FILE_RUNTIME_IGNORED, "runtime")
    if raw.get("version", 0) not in (0, CONFIG_VERSION):
        raise SystemExit(f"config {path} has unsupported version {raw['version']} (supported: {CONFIG_VERSION})")
    if raw.get("preset") and str(raw["preset"]).strip().lower() not in PRESETS:
        raise SystemExit("config preset: preset must be balanced, precise, creative, or deterministic")
    return raw


def apply_file_config(args, raw: dict) -> None:
    """What the file sets and no flag does: the order is defaults, the file's preset, the file's values,
    --preset, then the other flags (cmd/gopherllm/main.go:686-707, config.go:186-260)."""
    gen, run = raw.get("generation") or {}, raw.get("runtime") or {}
    if args.model is None and raw.get("model"):
        args.model = raw["model"]
    if args.max_tokens is None and gen.get("max_tokens") is not None:
        args.max_tokens = int(gen["max_tokens"])
    if args.seed is None and gen.get("seed") is not None:
        args.seed = int(gen["seed"])
    if args.stop is None and gen.get("stop") is not None:
        args.stop = [str(t) for t in gen["stop"]]
    if args.timeout is None and run.get("timeout") is not None:
        if parse_duration(str(run["timeout"])) <= 0:
            raise SystemExit("config runtime.timeout must be a duration greater than 0")
        args.timeout = str(run["timeout"])


def effective_sampler(args, file_config: dict = None) -> SamplerConfig:
    base = SamplerConfig()
    s = SamplerConfig(base.temperature, base.top_p, base.top_k, base.min_p, base.repeat_penalty)
    if file_config:
        if file_config.get("preset"):
            p = PRESETS[str(file_config["preset"]).strip().lower()]
            s = SamplerConfig(p.temperature, p.top_p, p.top_k, p.min_p, p.repeat_penalty)
        gen = file_config.get("generation") or {}
        for field in ("temperature", "top_p", "top_k", "min_p", "repeat_penalty"):
            if gen.get(field) is not None:
                setattr(s, field, int(gen[field]) if field == "top_k" else float(gen[field]))
    if args.preset:
        p = PRESETS[args.preset]
        s = SamplerConfig(p.temperature, p.top_p, p.top_k, p.min_p, p.repeat_penalty)
    for field, value in (("temperature", args.temp), ("top_p", args.top_p), ("top_k", args.top_k),
                         ("min_p", args.min_p), ("repeat_penalty", args.repeat_penalty)):
        if value is not None:
            setattr(s, field, value)
    return s


def inspect(path: str, list_metadata: bool, list_tensors: bool) -> int:
    """What --inspect prints (cmd/gopherllm/main.go:1182-1219), from config.json and
    the safetensors headers; no tensor data is read."""
    from .config import read_config_json
    from .config.registry import resolve_architecture
    from .weights.safetensors_io import index_folder
    raw = read_config_json(path)
    declared = (raw.get("architectures") or [raw.get("model_type", "")])[0]
    arch = resolve_architecture(declared) or resolve_architecture(raw.get("model_type", ""))
    shown = declared if arch is None or declared == arch.name else f"{declared} (loads as {arch.name})"
    entries = index_folder(path)
    print(f"file: {path}\nname: {raw.get('_name_or_path', '')}\narchitecture: {shown}\n"
          f"supported: {str(arch is not None).lower()}\nmetadata: {len(raw)}\ntensors: {len(entries)}")
    if list_metadata:
        for k in sorted(raw):
            print(f"{k:<48} {json.dumps(raw[k])}")
    if list_tensors:
        for name in sorted(entries):
            e = entries[name]
            print(f"{name:<56} {e.dtype:<8} dims={list(e.shape)} offset={e.begin}")
    return 0


def stats_line(s) -> str:
    tps = s.generated_tokens / max(1e-9, s.decode_time)
    return (f"prompt={s.prompt_tokens} generated={s.generated_tokens} ttft={s.ttft * 1e3:.0f}ms "
            f"prefill={s.prefill_time * 1e3:.0f}ms decode={s.decode_time * 1e3:.0f}ms "
            f"total={s.total_time * 1e3:.0f}ms tok/s={tps:.2f}")


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    file_config = load_file_config(args.config_file) if args.config_file else None
    if file_config:
        apply_file_config(args, file_config)
    if args.model is None:
        raise SystemExit("give a model folder (or \"model\" in the --config file)")
    args.max_tokens = 256 if args.max_tokens is None else args.max_tokens
    args.seed = 0 if args.seed is None else args.seed
    if args.random_config:
        from .api import write_random_model
        with open(args.random_config) as f:
            write_random_model(args.model, json.load(f), seed=args.seed)
        print(f"wrote {args.model}")
        return 0
    if args.inspect or args.list_tensors or args.list_metadata:
        return inspect(args.model, args.list_metadata, args.list_tensors)
    sampler = effective_sampler(args, file_config)
    if args.print_config:
        print(json.dumps({"model": args.model, "dtype": args.dtype, "max_tokens": args.max_tokens,
                          "seed": args.seed, "preset": args.preset or (file_config or {}).get("preset"), "sampler": vars(sampler),
                          "stop": args.stop, "timeout": args.timeout}, indent=2))
        return 0

    from .api import load
    log = (lambda m: print(m, file=sys.stderr, flush=True)) if args.verbose else None
    model = load(args.model, dtype=args.dtype, max_tokens=args.cache_tokens, device=args.device, log=log)
    if args.kernel_bench or args.kernel_bench_json:
        from .engine.kernel_bench import run_kernel_bench
        return run_kernel_bench(model, args.model, args.kernel_bench_runs, args.kernel_bench_layer,
                                args.kernel_bench_json)

    if args.prompt_file:
        with open(args.prompt_file) as f:
            prompts = [p for line in f if line.strip() for p in parse_prompts(line)]
    elif args.prompt:
        prompts = parse_prompts(args.prompt)
    elif args.bench or args.bench_json:
        import numpy as np
        rng = np.random.default_rng(args.seed or 1)
        prompts = [[int(t) for t in rng.integers(0, model.spec.vocab, size=min(64, model.spec.max_positions // 2))]]
    else:
        raise SystemExit("give --prompt or --prompt-file (token ids)")

    deadline = [None]
    timeout = parse_duration(args.timeout) if args.timeout else None
    opts = dict(max_tokens=args.max_tokens, sampler=sampler, seed=args.seed,
                should_stop=(lambda: deadline[0] is not None and time.monotonic() > deadline[0]))
    if args.stop is not None:
        opts["stop_tokens"] = [int(t) for t in args.stop]

    from .engine.generate import GenerationCanceled

    def one_run():
        deadline[0] = time.monotonic() + timeout if timeout else None
        try:
            return model.generate(prompts, **opts)
        except GenerationCanceled:
            raise SystemExit(f"generation timed out after {args.timeout}")

    if args.bench or args.bench_json:
        rows = []
        for i in range(args.bench_runs):
            for r in one_run():
                s = r.stats
                row = {"prompt_tokens": s.prompt_tokens, "generated_tokens": s.generated_tokens,
                       "ttft_ms": int(s.ttft * 1e3), "prefill_ms": int(s.prefill_time * 1e3),
                       "decode_ms": int(s.decode_time * 1e3), "total_ms": int(s.total_time * 1e3),
                       "prefill_tokens_per_second": s.prompt_tokens / max(1e-9, s.prefill_time),
                       "generated_tokens_per_second": s.generated_tokens / max(1e-9, s.decode_time)}
                if args.bench_output:
                    row["tokens"] = r.tokens
                rows.append(row)
                if not args.bench_json:
                    print(f"run {i + 1}: {stats_line(s)}")
                    if args.bench_output:
                        print(f"run {i + 1} output: {' '.join(map(str, r.tokens))}")
        if args.bench_json:
            print(json.dumps(rows))
        return 0

    if len(prompts) == 1:
        # one request: its tokens are printed as they come, as the reference streams its text
        opts["on_token"] = lambda i, tok: print(tok, end=" ", flush=True)
        r = one_run()[0]
        print()
        print(f"finish={r.finish_reason} {stats_line(r.stats)}", file=sys.stderr)
        return 0
    for r in one_run():
        print(" ".join(map(str, r.tokens)))
        print(f"finish={r.finish_reason} {stats_line(r.stats)}", file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
