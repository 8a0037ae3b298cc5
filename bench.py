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
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# Untimed decode steps between the prompts and the warm-up, the same whatever --warmup says.  After the
# prompts' products, which run at the power limit, the SM clock comes back in stages over about 35
# decode steps (90 ms; 3.05, 2.89, 2.68, 2.52, then 2.45 ms a step were measured): without them a figure
# would depend on how long ago the prompts ran, which is to say on the caller's --warmup.
SETTLE_STEPS = 40
SETTLE_POINT_MS = 150.0      # the least time the extra points (batch 1, batch 64) settle for before they are timed


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained") or 0.0)}, "measured"
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
    S = SETTLE_STEPS
    max_b = max(B, 64) if "points" in sections else B
    model = gl.load_random(cfg, seed=weight_seed, dtype="bfloat16", max_tokens=max_b * C, layers=layers)
    eng = model.engine
    spec = model.spec
    rng = np.random.default_rng(4)
    V = spec.vocab
    greedy = SamplerConfig.greedy()
    greedy_kw = dict(temperature=0.0, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, stop_tokens=(), seed=5)
    # bytes a decode step has to read: every matrix it uses once (the embedding table is only gathered
    # from) and the cached keys and values of the live sequences
    weight_bytes = sum(t.numel() * t.element_size() for t in eng.model._all_tensors()
                       if t is not None and t.dim() == 2) - eng.model.embedding.numel() * eng.model.embedding.element_size()
    kv_per_pos = eng.cache.bytes_per_position()

    def decode_rate(batch, steps, warmup, context, prompts=None, S=S):
        """`steps` on-device decode steps that end at `context` positions, after the prompts, S settling
        steps and `warmup` steps.  Returns tokens a second, ms a step, the mean cached length over the timed
        steps, and every token chosen after the prompts (the first from the prompts' logits)."""
        prompt_len = context - steps - warmup - S - 1
        if prompt_len < 1:
            raise SystemExit(f"context {context} is too short for {steps} + {warmup} + {S} steps")
        if prompts is None:
            prompts = [[int(t) for t in rng.integers(0, V, size=prompt_len)] for _ in range(batch)]
        slots = [eng.open() for _ in range(batch)]
        sampler = DeviceSampler(greedy, [request_seed(5, i) for i in range(batch)], prompts, V, eng.device)
        first = []
        for i in range(0, batch, 8):                       # fill the cache, 8 prompts a step
            rows = list(range(i, min(batch, i + 8)))
            logits = eng.step([(slots[j], prompts[j]) for j in rows])
            first += sampler.sample(logits, torch.tensor(rows, dtype=torch.int32).to(eng.device)).tolist()
        chosen = [first]
        toks = eng.decode_loop(slots, first, 1, sampler)   # captures the step
        chosen += toks.tolist()
        ops.LAUNCHES = 0
        if S + warmup > 1:
            toks = eng.decode_loop(slots, toks[-1].tolist(), S + warmup - 1, sampler)
            chosen += toks.tolist()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        toks = eng.decode_loop(slots, toks[-1].tolist(), steps, sampler)
        e1.record()
        torch.cuda.synchronize()
        eng.check_device()
        chosen += toks.tolist()
        ms = e0.elapsed_time(e1)
        ctx_mid = context - 1 - steps / 2.0
        for s in slots:
            eng.close(s)
        return batch * steps / (ms / 1e3), ms / steps, ctx_mid, chosen

    def point(batch, steps, context, settle_elsewhere=False):
        """One more decode measurement as a record: rate, time, bytes and the fraction of the HBM peak.
        ``settle_elsewhere``: the settling steps run on sequences of their own first, for a context too
        short to hold them."""
        # A point is taken right after other work (the prompts of 64 sequences, the prefill measurement) whose
        # power-capped clocks take a while to come back: it settles for SETTLE_POINT_MS at least, in steps
        # counted from the bytes a step reads, and says how many.
        est_ms = (weight_bytes + batch * context * kv_per_pos) / (0.6 * pk["hbm_gbs"] * 1e9) * 1e3
        settle = max(S, min(int(SETTLE_POINT_MS / est_ms), context // 4))
        if settle_elsewhere:
            decode_rate(batch, 1, 1, 8 + settle + 3, S=settle)
            rate, ms, mid, _ = decode_rate(batch, steps, 3, context, S=0)
        else:
            rate, ms, mid, _ = decode_rate(batch, steps, W, context, S=settle)
        nbytes = weight_bytes + batch * mid * kv_per_pos
        return {"value": round(rate, 1), "ms_per_step": round(ms, 4), "batch": batch, "context": context,
                "settle_steps": settle,
                "bytes": int(nbytes), "frac": round(nbytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4),
                "weights_only_frac": round(weight_bytes / (ms / 1e3) / 1e9 / pk["hbm_gbs"], 4)}

    prompt_len = C - K - W - S - 1
    prompts = [[int(t) for t in rng.integers(0, V, size=max(1, prompt_len))] for _ in range(B)]
    value, ms_step, ctx_mid, clock_info, launches_per_step, loop_tokens = 0.0, float("nan"), C - 1 - K / 2.0, {}, 0, None
    if "decode" in sections:
        clocks = ClockSampler()
        clocks.start()
        value, ms_step, ctx_mid, loop_tokens = decode_rate(B, K, W, C, prompts)
        clock_info = clocks.stop()
        launches_per_step = eng.launches_per_loop_step.get(B, 0)

    # the same work through the Python entry point: host tokens in, host tokens out
    e2e = None
    same_tokens = None
    if "e2e" in sections:
        model.generate(prompts, max_tokens=4, **greedy_kw)     # warm-up: captures the decode step for this batch
        res = model.generate(prompts, max_tokens=1 + S + W + K, **greedy_kw)
        # the S + W tokens after the prompt settle and warm up, as in the device-timed loop: the last K count
        dec_s = max(r.stats.token_times[-1] - (r.stats.token_times[-1 - K] if len(r.stats.token_times) > K
                                                 else r.stats.prefill_time) for r in res)
        e2e_value = B * K / dec_s
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": eng.h2d_bytes_last + 4 * B,
               "d2h_bytes_per_step": 4 * B}
        if loop_tokens is not None:
            # both figures come from one computation: the device loop chose the tokens the entry point chose
            n = min(len(loop_tokens), min(len(r.tokens) for r in res))
            same_tokens = all([row[i] for row in loop_tokens[:n]] == r.tokens[:n] for i, r in enumerate(res))
            if not same_tokens:
                raise SystemExit("bench: the on-device decode loop and Model.generate chose different tokens "
                                 "for the same prompts")
            e2e["same_tokens_as_device_loop"] = n

    step_bytes = weight_bytes + B * ctx_mid * kv_per_pos
    achieved = step_bytes / (ms_step / 1e3) / 1e9 if "decode" in sections else 0.0
    head_dim = spec.layers[0].mixer.head_dim
    out = {
        "metric": f"decode tok/s at batch {B}, context {C} ({label} sizes, bf16)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms_step, 4) if "decode" in sections else None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": f"synthetic: random weights N(0,0.02) seed {weight_seed}, token ids uniform in [0,51200)",
        "config": {"model": f"{label} sizes (PhiForCausalLM)", "layers": layers, "layers_of_model": layers_full,
                   "hidden": spec.hidden, "heads": spec.layers[0].mixer.num_heads,
                   "kv_heads": spec.layers[0].mixer.num_kv_heads, "head_dim": head_dim,
                   "intermediate": spec.layers[0].ffn.intermediate, "vocab": spec.vocab,
                   "rotary_dim": spec.layers[0].mixer.position.rotary_dim,
                   "global_batch": B, "seq_len": C,
                   "context_at_timed_steps": f"{C - K - 1}..{C - 1}", "settle_steps": S, "parallelism": "single GPU",
                   "sampling": "greedy", "l2": "each step reads weights and cache far larger than L2 (126 MB)",
                   "peaks": pk_src},
        "clocks": clock_info, "e2e": e2e, "gpu_launches": launches_per_step * K,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes": int(step_bytes),
                     "weights_only_frac": round(weight_bytes / (ms_step / 1e3) / 1e9 / pk["hbm_gbs"], 4)
                     if "decode" in sections else None},
    }
    # (the points before the prefill: its products run at the power limit, and a small decode step timed
    # right behind them is timed at clocks that are still coming back)
    if "points" in sections:
        detail = {"decode_b1": point(1, min(K, 64), C), "decode_b64": point(64, min(K, 32), C),
                  "decode_b64_ctx128": point(64, 16, 128, settle_elsewhere=True)}
        out["points"] = {"decode_b1": detail["decode_b1"]["value"], "decode_b64": detail["decode_b64"]["value"]}
        out["points_detail"] = detail
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
        eng.check_device()
        ms = min(times)
        layer_params = sum(w.numel() for e in spec.schedule for _, w, _, _ in eng.model.blocks[e.layer].products())
        flops = 2.0 * T * layer_params + 2.0 * T * T * spec.hidden * len(spec.schedule) + 2.0 * V * spec.hidden
        out["prefill"] = {"value": round(T / (ms / 1e3), 1), "tokens": T, "ms": round(ms, 3),
                          "frac": round(flops / (ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4),
                          "peak": "bf16_tflops (a burst of one product)", "flops": flops,
                          "frac_sustained": round(flops / (ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
                          if pk.get("bf16_tflops_sustained") else None}
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
