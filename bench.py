#!/usr/bin/env python3
"""Decode and prefill throughput of the liyab_b200 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--size small] [--layers L] [--dtype bfloat16]
    python bench.py --impl reference        # the reference's own tools on this machine's CPU, or why they cannot run

A step is one decode step of the whole batch.  The default run has the layer
sizes of GPT-2 small (12 layers, width 768, 12 heads) with random weights, a batch of
8 requests and the benchmark context of 1024 positions: 512-token prompts, then
decoding (contexts 512 -> 1024; when a request reaches the model's last position
its cache is cut back to the prompt and decoding goes on, so any K can be timed).
`value` is decoded tokens per second timed with CUDA events over exactly K
steps (the library's own measurement, host/bench.cpp: the engine's step function,
sampling on the device, ids fed back without leaving it); `e2e` is the same through
the Python entry point (Engine.generate_batch: host token ids in, host token ids
out, per-step copies both ways included).  One JSON line is printed.  Beside the
headline it holds: `points` (batch 1 and 64) with `points_detail`, `prefill`
(2 x 1024 tokens), `roofline`, `fp32` (the 32-bit engine), `medium` and `xl`
(the other two GPT-2 sizes at their full layer counts), `mixed_xl` (64 requests
with prompts of 1..1024 tokens generated to position 1024 through the scheduler)
and `same` (the timed end-to-end run's tokens equal an untimed run's).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GPT2_SMALL = dict(model_type="gpt2", n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                  n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new",
                  scale_attn_by_inverse_layer_idx=False, tie_word_embeddings=True)
SIZES = {"small": GPT2_SMALL,
         "medium": dict(GPT2_SMALL, n_layer=24, n_embd=1024, n_head=16, n_inner=4096),
         "xl": dict(GPT2_SMALL, n_layer=48, n_embd=1600, n_head=25, n_inner=6400)}
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
FP32_TFLOPS_NOMINAL = 80.0          # 32-bit units, no tensor cores; no measured figure exists for it


def peaks():
    """Measured denominators if the driver wrote them, else the stated fallback."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            raw = json.load(f)
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])), "source": "measured"}
    except (OSError, KeyError, ValueError):
        return dict(FALLBACK_PEAKS, bf16_tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "20"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        mhz = sorted(int(r[0]) for r in self.rows if r and r[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 6 for n, v in zip(names, r[2:6]) if v.lower().startswith("active")})
        mx = next((int(r[1]) for r in self.rows if len(r) > 1 and r[1].isdigit()), None)
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": reasons, "samples": len(mhz)}


def model_bytes_and_flops(cfg, dtype_bytes):
    d, ff, V, L = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"], cfg["n_layer"]
    per_layer = 4 * d * d + 2 * d * ff
    weight_bytes = dtype_bytes * (L * per_layer + V * d)        # every matrix once; the tied table once
    kv_per_pos = 2 * L * d * dtype_bytes

    def prefill_flops(seq_lens, rows):
        T = sum(seq_lens)
        return 2 * T * L * per_layer + sum(2 * L * d * s * s for s in seq_lens) + 2 * rows * V * d

    return weight_bytes, kv_per_pos, prefill_flops


def decode_point(replayer, cfg, dtype_bytes, batch, steps, warmup, pk, seed=0):
    """One device-timed decode measurement with its roofline fraction."""
    r = replayer.bench_decode(batch, PROMPT_LEN, steps, warmup, seed)
    weight_bytes, kv_per_pos, _ = model_bytes_and_flops(cfg, dtype_bytes)
    step_bytes = weight_bytes + batch * r["mean_context"] * kv_per_pos
    achieved = step_bytes / (r["ms_per_step"] / 1e3) / 1e9
    r.update(tok_s=batch / (r["ms_per_step"] / 1e3), step_bytes=step_bytes, achieved_gbs=achieved, frac=achieved / pk["hbm_gbs"])
    return r


def prefill_point(replayer, cfg, dtype_bytes, pk, dtype):
    n_seq = PREFILL_TOKENS // 1024
    r = replayer.bench_prefill(n_seq, 1024, 5)
    _, _, flops = model_bytes_and_flops(cfg, dtype_bytes)
    peak = pk["bf16_tflops"] if dtype == "bfloat16" else FP32_TFLOPS_NOMINAL
    ms = r["ms_per_step"]
    return {"value": round(PREFILL_TOKENS / (ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 4),
            "frac": round(flops([1024] * n_seq, n_seq) / (ms / 1e3) / 1e12 / peak, 4), "median_ms": round(r["wall_ms_per_step"], 4),
            "launches": r["kernel_launches"]}


def detail(r):
    return {"tokens_per_s": round(r["tok_s"], 1), "ms_per_step": round(r["ms_per_step"], 4), "mean_context": round(r["mean_context"], 1),
            "frac": round(r["frac"], 4), "path": "fused" if r["fused_steps"] else ("graph" if r["graph_steps"] else "parts")}


def e2e_run(model_dir, dtype, batch, steps):
    """The same metric through Engine.generate_batch: host ids in, host ids out.  The workload runs twice (the first,
    untimed, also warms the engine up); `same` says that both runs gave the same tokens."""
    import numpy as np
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine(EngineConfig(model=model_dir, dtype=dtype, max_requests=batch, max_batched_tokens=2048,
                                 num_pages=batch * 64, cuda_graphs=True))
    rng = np.random.default_rng(2)
    n_new = min(steps, engine.max_positions - PROMPT_LEN)
    prompts = [rng.integers(0, engine.vocab_size, size=PROMPT_LEN).tolist() for _ in range(batch)]
    params = SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True)
    untimed = engine.generate_batch(prompts, params)
    before = engine.stats()
    results = engine.generate_batch(prompts, params)
    after = engine.stats()
    decode_ms = max(r.stats.decode_ms for r in results)
    tokens = sum(max(0, r.stats.generated_tokens - 1) for r in results)
    n_steps = max(1, after["steps"] - before["steps"])
    out = {"value": round(tokens / (decode_ms / 1e3), 1) if decode_ms > 0 else 0.0, "unit": "tokens/s",
           "h2d_bytes_per_step": (after["h2d_bytes"] - before["h2d_bytes"]) // n_steps,
           "d2h_bytes_per_step": (after["d2h_bytes"] - before["d2h_bytes"]) // n_steps, "steps": n_new}
    same = [r.tokens for r in results] == [r.tokens for r in untimed]
    engine.close()
    return out, same


def mixed_run(model_dir, dtype, n_requests, budget):
    """64 requests with prompts of 1..positions tokens, each generated to the model's last position, all submitted at
    once: chunked prefill beside decoding through the scheduler; host ids in and out."""
    import numpy as np
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine(EngineConfig(model=model_dir, dtype=dtype, max_requests=n_requests, max_batched_tokens=budget, page_size=16))
    P = engine.max_positions
    rng = np.random.default_rng(3)
    lens = rng.integers(1, P + 1, size=n_requests)
    prompts = [rng.integers(0, engine.vocab_size, size=int(k)).tolist() for k in lens]
    params = [SamplingParams(temperature=0.0, max_tokens=max(1, int(P - k)), ignore_eos=True) for k in lens]
    engine.generate_batch([p[:8] for p in prompts[:4]], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    before = engine.stats()
    t0 = time.perf_counter()
    results = engine.generate_batch(prompts, params)
    seconds = time.perf_counter() - t0
    after = engine.stats()
    generated = sum(r.stats.generated_tokens for r in results)
    out = {"requests": n_requests, "prompt_tokens": int(lens.sum()), "generated_tokens": generated, "seconds": round(seconds, 3),
           "generated_tokens_per_s": round(generated / seconds, 1), "total_tokens_per_s": round((generated + int(lens.sum())) / seconds, 1),
           "steps": after["steps"] - before["steps"], "preemptions": after["preemptions"] - before["preemptions"],
           "batched_token_histogram": {k: a - b for k, a, b in zip(["1", "2-8", "9-32", "33-128", "129-512", "513-2048", ">2048"],
                                                                   after["histogram"], before["histogram"])},
           "finished": sorted({r.finish_reason for r in results}), "page_size": 16, "token_budget": budget}
    engine.close()
    return out


def size_block(tmp, size, dtype, steps, pk):
    """Decode at batch 1 / 8 / 64 and the 2,048-token prefill of one GPT-2 size at its full layer count."""
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import write_random_model
    cfg = SIZES[size]
    dtype_bytes = 2 if dtype == "bfloat16" else 4
    folder = write_random_model(os.path.join(tmp, f"gpt2_{size}_{dtype}"), cfg, seed=0, dtype=dtype)
    rep = Replayer(folder, dtype, max_tokens=64 * 1024, max_requests=64, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
    block = {"n_layer": cfg["n_layer"], "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"]}
    for b in (1, 8, 64):
        block[f"decode_b{b}"] = detail(decode_point(rep, cfg, dtype_bytes, b, steps, 3, pk))
    block["prefill"] = prefill_point(rep, cfg, dtype_bytes, pk, dtype)
    rep.close()
    return block, folder


def reference_arm(args) -> int:
    from baseline.reference_arm import run
    return run(args)


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--size", default="small", choices=sorted(SIZES), help="the model of the headline figures")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (reported)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="the headline figure only")
    ap.add_argument("--no-extra", action="store_true", help="skip the 32-bit engine, the other sizes and the mixed workload")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    args.warmup = max(args.warmup, 3)
    from liyab_b200.engine import Replayer
    from liyab_b200.weights import write_random_model
    full = SIZES[args.size]
    cfg = dict(full, n_layer=args.layers or full["n_layer"])
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    pk = peaks()
    with tempfile.TemporaryDirectory(prefix="liyab_b200_bench_") as tmp:
        model_dir = write_random_model(os.path.join(tmp, f"gpt2_{args.size}"), cfg, seed=0, dtype=args.dtype)
        big = max(64, args.batch)
        rep = Replayer(model_dir, args.dtype, max_tokens=big * 1024, max_requests=big, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
        decode_point(rep, cfg, dtype_bytes, args.batch, 20, args.warmup, pk)          # loads and warms everything up
        clocks = ClockSampler()
        clocks.start()
        main_run = decode_point(rep, cfg, dtype_bytes, args.batch, args.steps, args.warmup, pk)
        clock_info = clocks.stop()
        line = {
            "metric": f"GPT-2 {args.size} decode tokens/s (batch {args.batch}, 512-token prompts, contexts 512-1024)",
            "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
            "data": "synthetic: uniform random token ids, random-init weights (seed 0)",
            "config": {"model": f"gpt2-{args.size}", "n_layer": cfg["n_layer"], "n_layer_full": full["n_layer"], "n_embd": cfg["n_embd"],
                       "n_head": cfg["n_head"], "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"],
                       "n_positions": cfg["n_positions"], "global_batch": args.batch, "seq_len": 1024,
                       "prompt_len": PROMPT_LEN, "mean_context": round(main_run["mean_context"], 1), "page_size": 16,
                       "parallelism": "single-gpu", "l2": "each step reads %.0f MB of weights and cache > 126 MB L2" % (main_run["step_bytes"] / 1e6),
                       "peaks": pk["source"], "decode_path": detail(main_run)["path"], "host": "C++ library through its C interface"},
            "gpu_launches": main_run["kernel_launches"],
            "roofline": {"bound": "hbm", "achieved": round(main_run["achieved_gbs"], 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(main_run["frac"], 4)},
            "clocks": clock_info,
        }
        if not args.no_points:
            points, details = {}, {}
            for b in (1, 64):
                r = decode_point(rep, cfg, dtype_bytes, b, min(args.steps, 256), 3, pk)
                points[f"decode_b{b}"] = round(r["tok_s"], 1)
                details[f"decode_b{b}"] = detail(r)
            line["points"] = points
            line["points_detail"] = details
            line["prefill"] = prefill_point(rep, cfg, dtype_bytes, pk, args.dtype)
            rep.close()
            line["e2e"], line["same"] = e2e_run(model_dir, args.dtype, args.batch, args.steps)
        else:
            rep.close()
        if not args.no_points and not args.no_extra:
            steps = min(args.steps, 64)
            other = "float32" if args.dtype == "bfloat16" else "bfloat16"
            if other == "float32":
                folder = write_random_model(os.path.join(tmp, "gpt2_small_f32"), SIZES["small"], seed=0, dtype="float32")
                rep32 = Replayer(folder, "float32", max_tokens=8 * 1024, max_requests=8, cuda_graphs=True, max_step_tokens=PREFILL_TOKENS)
                line["fp32"] = {"model": "gpt2-small", "decode_b8": detail(decode_point(rep32, SIZES["small"], 4, 8, steps, 3, pk)),
                                "prefill": prefill_point(rep32, SIZES["small"], 4, pk, "float32"),
                                "note": "true 32-bit: FMA products, float32 cache; prefill frac against %g TFLOP/s nominal" % FP32_TFLOPS_NOMINAL}
                rep32.close()
            for size in ("medium", "xl"):
                if size == args.size:
                    continue
                block, folder = size_block(tmp, size, args.dtype, steps, pk)
                line[size] = block
                if size == "xl":
                    line["mixed_xl"] = mixed_run(folder, args.dtype, 64, 2048)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
