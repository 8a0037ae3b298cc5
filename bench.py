#!/usr/bin/env python3
"""Decode and prefill throughput of the Phi-2 sized model with random weights on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--context 2048] [--layers L]
    python bench.py --model phi-1.5          the same measurements at Phi-1.5's layer sizes
    python bench.py --ragged                 64 unequal prompts as one batch through Model.generate

Prints one JSON line.  ``value`` is decoded tokens a second at the given batch and
context, timed on the device over K decode steps that run back to back without the
host (each step feeds the tokens the step before chose); ``e2e`` is the same work
through the Python entry point ``Model.generate``, with host token lists in and out,
every step copying its descriptor from pinned host memory and reading the chosen
tokens back.  ``prefill`` is one prompt of 2,048 tokens; ``points`` are decode rates at
batch 1 and 64; ``roofline`` relates the decode step to the bytes it has to read.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Phi-2 sizes: the layer sizes of the benchmark configuration
PHI2 = dict(architectures=["PhiForCausalLM"], model_type="phi", num_hidden_layers=32, hidden_size=2560,
            num_attention_heads=32, num_key_value_heads=32, intermediate_size=10240, vocab_size=51200,
            partial_rotary_factor=0.4, rope_theta=10000.0, layer_norm_eps=1e-5, hidden_act="gelu_new",
            qk_layernorm=False, tie_word_embeddings=False, max_position_embeddings=2048,
            initializer_range=0.02, torch_dtype="bfloat16")
# Phi-1.5 sizes (Phi-1 has the same layer shapes)
PHI15 = dict(PHI2, num_hidden_layers=24, hidden_size=2048, intermediate_size=8192, partial_rotary_factor=0.5)
MODELS = {"phi-2": ("Phi-2", PHI2, 2), "phi-1.5": ("Phi-1.5", PHI15, 3)}      # label, sizes, seed of the weights
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"])}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    # After the prompts' products, which run at the power limit, the SM clock comes back in steps over
    # about 35 decode steps (90 ms; 3.05, 2.89, 2.68, 2.52, then 2.45 ms a step were measured): the
    # default warm-up covers that, for the device-timed loop and for the end-to-end run alike.
    ap.add_argument("--warmup", type=int, default=40)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048, help="positions each sequence holds when the timed steps end")
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the configuration has")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--skip-points", action="store_true", help="leave out prefill, batch 1 and batch 64")
    ap.add_argument("--sections", default="decode,e2e,prefill,points",
                    help="which measurements to run (for profiling a part): decode,e2e,prefill,points")
    ap.add_argument("--model", default="phi-2", choices=sorted(MODELS), help="whose layer sizes to run")
    ap.add_argument("--ragged", action="store_true",
                    help="instead: 64 prompts of 16..1536 tokens as one batch through Model.generate, 512 tokens "
                         "each at temperature 0.8, and a 32-bit check of 4 of them")
    args = ap.parse_args()

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "SimonWaldherr/GopherLLM is a Go module (no setup.py/pyproject.toml; pip reports 'not "
                          "installable') and no Go toolchain exists offline, so it cannot be built or run here"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures one GPU: this library has no multi-GPU path (asked for {args.gpus})")
        return 2
    if args.warmup < 3:
        args.warmup = 3
    sections = set(args.sections.split(","))
    if args.skip_points:
        sections -= {"prefill", "points"}

    import numpy as np
    import torch
    import gopherllm_b200 as gl
    from gopherllm_b200 import ops
    from gopherllm_b200.sampling.sampler import DeviceSampler, SamplerConfig, request_seed

    pk, pk_src = peaks()
    label, sizes, weight_seed = MODELS[args.model]
    cfg = dict(sizes)
    layers_full = cfg["num_hidden_layers"]
    layers = args.layers or layers_full
    if args.ragged:
        return ragged(args, label, cfg, weight_seed, layers, layers_full)
    K, W, B, C = args.steps, args.warmup, args.batch, args.context
    max_b = max(B, 64) if "points" in sections else B
    model = gl.load_random(cfg, seed=weight_seed, dtype="bfloat16", max_tokens=max_b * C, layers=layers)
    eng = model.engine
    spec = model.spec
    rng = np.random.default_rng(4)
    V = spec.vocab
    greedy = SamplerConfig.greedy()
    weight_bytes = sum(t.numel() * t.element_size() for t in eng.model._all_tensors()
                       if t is not None and t.dim() == 2) - eng.model.embedding.numel() * eng.model.embedding.element_size()
    kv_per_pos = eng.cache.bytes_per_position()

    def decode_rate(batch, steps, warmup, context):
        """tokens a second of `steps` on-device decode steps ending at `context` positions."""
        prompt_len = context - steps - warmup - 1
        prompts = [[int(t) for t in rng.integers(0, V, size=prompt_len)] for _ in range(batch)]
        slots = [eng.open() for _ in range(batch)]
        sampler = DeviceSampler(greedy, [request_seed(5, i) for i in range(batch)], prompts, V, eng.device)
        for i in range(0, batch, 8):                       # fill the cache, 8 prompts a step
            logits = eng.step([(slots[j], prompts[j]) for j in range(i, min(batch, i + 8))])
        first = [int(t) for t in rng.integers(0, V, size=batch)]
        eng.decode_loop(slots, first, 1, sampler)          # captures the step
        ops.LAUNCHES = 0
        toks = eng.decode_loop(slots, first, warmup, sampler)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks = eng.decode_loop(slots, toks[-1].tolist(), steps, sampler)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        ctx_mid = context - 1 - steps / 2.0
        for s in slots:
            eng.close(s)
        return batch * steps / (ms / 1e3), ms / steps, ctx_mid

    value, ms_step, ctx_mid, clock_info, launches_per_step = 0.0, float("nan"), C - 1 - K / 2.0, {}, 0
    if "decode" in sections:
        clocks = ClockSampler()
        clocks.start()
        value, ms_step, ctx_mid = decode_rate(B, K, W, C)
        clock_info = clocks.stop()
        launches_per_step = eng.launches_per_loop_step.get(B, 0)

    # the same work through the Python entry point: host tokens in, host tokens out
    e2e = None
    if "e2e" in sections:
        prompt_len = C - K - W - 1
        prompts = [[int(t) for t in rng.integers(0, V, size=prompt_len)] for _ in range(B)]
        model.generate(prompts[:B], max_tokens=4, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                       stop_tokens=(), seed=5)             # warm-up: captures the decode step for this batch
        res = model.generate(prompts, max_tokens=K + W, temperature=0.0, top_k=0, top_p=1.0, repeat_penalty=1.0,
                             stop_tokens=(), seed=5)
        # the W tokens after the prompt are warm-up, as in the device-timed loop: the last K count
        dec_s = max(r.stats.token_times[-1] - (r.stats.token_times[-1 - K] if len(r.stats.token_times) > K
                                                 else r.stats.prefill_time) for r in res)
        e2e_value = B * K / dec_s
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": eng.h2d_bytes_last + 4 * B,
               "d2h_bytes_per_step": 4 * B}

    step_bytes = weight_bytes + B * ctx_mid * kv_per_pos
    achieved = step_bytes / (ms_step / 1e3) / 1e9 if "decode" in sections else 0.0
    out = {
        "metric": f"decode tok/s at batch {B}, context {C} ({label} sizes, bf16)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4) if "decode" in sections else None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": f"synthetic: random weights N(0,0.02) seed {weight_seed}, token ids uniform in [0,51200)",
        "config": {"model": f"{label} sizes (PhiForCausalLM)", "layers": layers, "layers_of_model": layers_full,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["hidden_size"] // cfg["num_attention_heads"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
                   "rotary_dim": int(cfg["partial_rotary_factor"] * (cfg["hidden_size"] // cfg["num_attention_heads"])),
                   "global_batch": B, "seq_len": C,
                   "context_at_timed_steps": f"{C - K - 1}..{C - 1}", "parallelism": "single GPU",
                   "sampling": "greedy", "l2": "each step reads weights and cache far larger than L2 (126 MB)",
                   "peaks": pk_src},
        "clocks": clock_info, "e2e": e2e, "gpu_launches": launches_per_step * K,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if "prefill" in sections:
        T = 2048
        toks = [int(t) for t in rng.integers(0, V, size=T)]
        s = eng.open()
        eng.step([(s, toks)])                              # warm-up
        eng.close(s)
        times = []
        for _ in range(3):
            s = eng.open()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            eng.step([(s, toks)])
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
            eng.close(s)
        ms = min(times)
        layer_params = sum(w.numel() for e in spec.schedule for _, w, _, _ in eng.model.blocks[e.layer].products())
        flops = 2.0 * T * layer_params + 2.0 * T * T * cfg["hidden_size"] * layers + 2.0 * V * cfg["hidden_size"]
        out["prefill"] = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                          "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
    if "points" in sections:
        b1, _, _ = decode_rate(1, min(K, 64), W, C)
        b64, _, _ = decode_rate(64, min(K, 32), W, C)
        out["points"] = {"decode_b1": round(b1, 1), "decode_b64": round(b64, 1)}
    print(json.dumps(out))
    return 0


def ragged(args, label, cfg, weight_seed, layers, layers_full):
    """A batch of unequal prompts through the entry point: 64 sequences that start together, lengths uniform
    in [16, 1536] (seed 4), one step for all prompts, then 512 tokens each at temperature 0.8 (seed 5); and
    the last prompt position's logits of 4 of the sequences in bfloat16 against the 32-bit path."""
    import numpy as np
    import torch
    import gopherllm_b200 as gl
    B, N, n_check = 64, 512, 4
    rng = np.random.default_rng(4)
    V = cfg["vocab_size"]
    lens = [int(n) for n in rng.integers(16, 1537, size=B)]
    prompts = [[int(t) for t in rng.integers(0, V, size=n)] for n in lens]
    model = gl.load_random(cfg, seed=weight_seed, dtype="bfloat16", max_tokens=B * 2048, layers=layers)
    opts = dict(max_tokens=N, temperature=0.8, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0,
                stop_tokens=(), seed=5)
    model.generate(prompts, **opts)                        # warm-up: loads the kernels, captures the steps
    clocks = ClockSampler()
    clocks.start()
    res = model.generate(prompts, **opts)
    clock_info = clocks.stop()
    generated = sum(r.stats.generated_tokens for r in res)
    prefill_s = max(r.stats.prefill_time for r in res)
    total_s = max(r.stats.total_time for r in res)
    # 32-bit check: the logits after the prompt, for the first sequences, both ways
    eng = model.engine
    got = []
    for p in prompts[:n_check]:
        s = eng.open()
        got.append(eng.step([(s, p)])[0].float().cpu())
        eng.close(s)
    model.close()
    del model, eng
    torch.cuda.empty_cache()
    m32 = gl.load_random(cfg, seed=weight_seed, dtype="float32", max_tokens=2048, layers=layers)
    diff, scale, same = 0.0, 0.0, 0
    for p, g in zip(prompts[:n_check], got):
        s = m32.engine.open()
        want = m32.engine.step([(s, p)])[0].cpu()
        m32.engine.close(s)
        diff = max(diff, float((g - want).abs().max()))
        scale = max(scale, float(want.abs().max()))
        same += int(int(g.argmax()) == int(want.argmax()))
    print(json.dumps({
        "metric": f"generated tok/s of a ragged batch of {B} ({label} sizes, bf16, through Model.generate)",
        "value": round(generated / (total_s - prefill_s), 1), "unit": "tokens/s", "n_gpus": 1,
        "higher_is_better": True, "dtype": "bf16",
        "data": f"synthetic: random weights N(0,0.02) seed {weight_seed}, prompt lengths uniform in [16,1536] seed 4, "
                "token ids uniform in [0,51200), temperature 0.8 seed 5",
        "config": {"model": f"{label} sizes (PhiForCausalLM)", "layers": layers, "layers_of_model": layers_full,
                   "global_batch": B, "prompt_tokens": sum(lens), "longest_prompt": max(lens),
                   "new_tokens_each": N, "cache_positions_per_slot": 2048, "timing": "host clock around the entry point"},
        "generated_tokens": generated, "decode_s": round(total_s - prefill_s, 4),
        "prefill": {"tokens": sum(lens), "ms": round(prefill_s * 1e3, 2), "value": round(sum(lens) / prefill_s, 1)},
        "clocks": clock_info,
        "fp32_check": {"sequences": n_check, "max_abs_diff": round(diff, 5), "max_abs_logit": round(scale, 4),
                       "argmax_equal": same},
    }))
    return 0


if __name__ == "__main__":
    sys.exit(main())
