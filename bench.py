#!/usr/bin/env python3
"""Decode and prefill throughput of the liyab_b200 engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--batch 8] [--layers L] [--dtype bfloat16]
    python bench.py --impl reference        # prints why the reference cannot run here

A step is one decode step of the whole batch.  The default run has the layer
sizes of GPT-2 small (12 layers, width 768, 12 heads) with random weights, a batch of
8 requests and the benchmark context of 1024 positions: 512-token prompts, then
decoding (contexts 512 -> 1024; when a request reaches the model's last position
its cache is cut back to the prompt and decoding goes on, so any K can be timed).
`value` is decoded tokens per second timed with CUDA events over exactly K
steps; `e2e` is the same through the Python entry point (Engine.generate_batch:
host token ids in, host token ids out, per-step copies both ways included).
One JSON line is printed; see the keys below.
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
FULL_LAYERS = GPT2_SMALL["n_layer"]
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


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


def model_bytes_and_flops(cfg, n_layers, dtype_bytes):
    d, ff, V = cfg["n_embd"], cfg["n_inner"], cfg["vocab_size"]
    per_layer = 4 * d * d + 2 * d * ff
    weight_bytes = dtype_bytes * (n_layers * per_layer + V * d)        # every matrix once; the tied table once
    kv_per_pos = 2 * n_layers * d * dtype_bytes

    def prefill_flops(seq_lens, rows):
        T = sum(seq_lens)
        return 2 * T * n_layers * per_layer + sum(2 * n_layers * d * s * s for s in seq_lens) + 2 * rows * V * d

    return weight_bytes, kv_per_pos, prefill_flops


def decode_run(model_dir, dtype, batch, steps, warmup, clocks=None):
    """Device-timed decode: K steps of `batch` requests after 512-token prompts; returns a dict of measurements."""
    import numpy as np
    import torch
    from liyab_b200 import ops
    from liyab_b200.engine import StepEntry
    from liyab_b200.engine.replay import build_replayer
    from liyab_b200.sampling.params import SamplingParams
    from liyab_b200.sampling.sampler import DeviceSampler

    model, cache, stepper = build_replayer(model_dir, dtype, max_tokens=batch * 1024, page_size=16, max_requests=batch)
    stepper.cuda_graphs = True
    stepper.workspace.reserve_rows(max(PREFILL_TOKENS, batch))
    P, V = model.max_positions, model.spec.vocab_size
    rng = np.random.default_rng(0)
    sampler = DeviceSampler(model.runtime.device, batch)
    greedy = [SamplingParams(temperature=0.0)] * batch
    ids = [f"b{i}" for i in range(batch)]
    for r in ids:                       # prompts, two at a time (2 x 512 tokens a step)
        cache.open(r)
    for i in range(0, batch, 2):
        chunk = ids[i:i + 2]
        out = stepper.step([StepEntry(r, rng.integers(0, V, size=PROMPT_LEN).tolist(), [PROMPT_LEN - 1]) for r in chunk])
    sampler.out_ids[:batch].fill_(1)      # any valid ids start the decode loop; from then on they are the sampled ones
    ctx_sum, launches = 0, 0

    from liyab_b200.engine.step import DeviceTokens
    identity = list(range(batch))
    pending = [None]

    def one_step():
        """One decode step the way the engine runs it: the ids of the step before stay on the device and feed
        this step; they are copied to the host while this step computes, and waited for after it is launched."""
        nonlocal ctx_sum
        if cache.length(ids[0]) + 1 > P:
            for r in ids:
                cache.truncate(r, PROMPT_LEN)
        ctx_sum += sum(cache.length(r) + 1 for r in ids)
        out = stepper.step([StepEntry(r, [0], [0]) for r in ids], DeviceTokens(sampler.out_ids, identity))
        sampler.sample(out.logits, greedy, [0.0] * batch)
        ticket = sampler.fetch_async(batch)
        if pending[0] is not None:
            sampler.wait(pending[0], batch)
        pending[0] = ticket

    for _ in range(warmup):
        one_step()
    if clocks is not None:          # clocks are sampled while the timed steps run, not while the model loads
        clocks.start()
        for _ in range(max(warmup, 20)):
            one_step()
    ctx_sum = 0
    ops.LAUNCHES = 0
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        one_step()
    sampler.wait(pending[0], batch)
    pending[0] = None
    end.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    ms = start.elapsed_time(end)
    clock_info = clocks.stop() if clocks is not None else None
    per_graph = getattr(stepper, "graph_launches", {}).get(batch, 0)
    launches = ops.LAUNCHES + per_graph * steps
    for r in ids:
        cache.close(r)
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "mean_ctx": ctx_sum / (steps * batch),
            "launches": launches, "wall_ms_per_step": wall_ms / steps, "weight_bytes": model.weight_bytes(),
            "clocks": clock_info, "fused_steps": stepper.fused_steps, "graph_steps": stepper.graph_steps}


def prefill_run(model_dir, dtype, repeats=5):
    import numpy as np
    import torch
    from liyab_b200.engine import StepEntry
    from liyab_b200.engine.replay import build_replayer
    model, cache, stepper = build_replayer(model_dir, dtype, max_tokens=4096, page_size=16)
    stepper.cuda_graphs = True              # as the engine runs it: a step of a shape seen before replays its graph
    stepper.workspace.reserve_rows(PREFILL_TOKENS)
    V = model.spec.vocab_size
    rng = np.random.default_rng(1)
    n_seq = PREFILL_TOKENS // 1024
    best = None
    for it in range(repeats + 2):
        for i in range(n_seq):
            cache.open(f"p{i}")
        entries = [StepEntry(f"p{i}", rng.integers(0, V, size=1024).tolist(), [1023]) for i in range(n_seq)]
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        stepper.step(entries)
        e.record()
        torch.cuda.synchronize()
        if it >= 2:
            best = min(best or 1e30, s.elapsed_time(e))
        for i in range(n_seq):
            cache.close(f"p{i}")
    return best


def e2e_run(model_dir, dtype, batch, steps):
    """The same metric through Engine.generate_batch: host ids in, host ids out."""
    import numpy as np
    from liyab_b200 import Engine, EngineConfig, SamplingParams
    engine = Engine(EngineConfig(model=model_dir, dtype=dtype, max_requests=batch, max_batched_tokens=2048,
                                 num_pages=batch * 64, cuda_graphs=True))
    V = engine.model.spec.vocab_size
    rng = np.random.default_rng(2)
    n_new = min(steps, engine.max_positions - PROMPT_LEN)
    prompts = [rng.integers(0, V, size=PROMPT_LEN).tolist() for _ in range(batch)]
    engine.generate_batch([p[:32] for p in prompts], SamplingParams(temperature=0.0, max_tokens=8, ignore_eos=True))  # warm-up
    results = engine.generate_batch(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    decode_ms = max(r.stats.decode_ms for r in results)
    tokens = sum(max(0, r.stats.generated_tokens - 1) for r in results)
    width = (engine.max_positions + 15) // 16
    h2d = 4 * (7 * batch + 1 + batch * width + batch) + 24 * batch      # layout arrays + block table + sampler options
    return {"value": tokens / (decode_ms / 1e3) if decode_ms > 0 else 0.0, "unit": "tokens/s",
            "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * batch, "steps": n_new}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=FULL_LAYERS, help="fewer layers than the configuration (reported)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 / 64, prefill and the end-to-end run")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": "liyab is a CMake C++ CPU/Metal/Vulkan engine with no Python "
                          "package (pip: neither setup.py nor pyproject.toml found) and no CUDA code; it cannot run on a B200"}))
        return 0
    if args.gpus != 1:
        print(f"bench.py measures a single-GPU engine; --gpus {args.gpus} is not supported (run with --gpus 1)")
        return 2
    args.warmup = max(args.warmup, 3)
    import torch
    from liyab_b200.config import parse_config
    from liyab_b200.weights import write_random_model
    cfg = dict(GPT2_SMALL, n_layer=args.layers)
    dtype_bytes = 2 if args.dtype == "bfloat16" else 4
    pk = peaks()
    with tempfile.TemporaryDirectory(prefix="liyab_b200_bench_") as tmp:
        model_dir = write_random_model(os.path.join(tmp, "gpt2_small"), parse_config(cfg), seed=0, dtype=args.dtype)
        main_run = decode_run(model_dir, args.dtype, args.batch, args.steps, args.warmup, clocks=ClockSampler())
        clock_info = main_run["clocks"]
        weight_bytes, kv_per_pos, prefill_flops = model_bytes_and_flops(cfg, args.layers, dtype_bytes)
        step_bytes = weight_bytes + args.batch * main_run["mean_ctx"] * kv_per_pos
        achieved = step_bytes / (main_run["ms_per_step"] / 1e3) / 1e9
        line = {
            "metric": "GPT-2 small decode tokens/s (batch 8, 512-token prompts, contexts 512-1024)",
            "value": round(main_run["tok_s"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if args.dtype == "bfloat16" else "fp32",
            "data": "synthetic: uniform random token ids, random-init weights (seed 0)",
            "config": {"model": "gpt2-small", "n_layer": args.layers, "n_layer_full": FULL_LAYERS, "n_embd": cfg["n_embd"],
                       "n_head": cfg["n_head"], "n_inner": cfg["n_inner"], "vocab_size": cfg["vocab_size"],
                       "n_positions": cfg["n_positions"], "global_batch": args.batch, "seq_len": 1024,
                       "prompt_len": PROMPT_LEN, "mean_context": round(main_run["mean_ctx"], 1), "page_size": 16,
                       "parallelism": "single-gpu", "l2": "each step reads %.0f MB of weights and cache > 126 MB L2" % (step_bytes / 1e6),
                       "peaks": pk["source"], "decode_path": "fused" if main_run["fused_steps"] else "graph"},
            "gpu_launches": main_run["launches"],
            "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": round(achieved / pk["hbm_gbs"], 4)},
            "clocks": clock_info,
        }
        if not args.no_points:
            points = {}
            for b in (1, 64):
                points[f"decode_b{b}"] = round(decode_run(model_dir, args.dtype, b, min(args.steps, 256), 3)["tok_s"], 1)
            line["points"] = points
            ms = prefill_run(model_dir, args.dtype)
            flops = prefill_flops([1024] * (PREFILL_TOKENS // 1024), PREFILL_TOKENS // 1024)
            peak = pk["bf16_tflops"] if args.dtype == "bfloat16" else 80.0
            line["prefill"] = {"value": round(PREFILL_TOKENS / (ms / 1e3), 1), "tokens": PREFILL_TOKENS, "ms": round(ms, 4),
                               "frac": round(flops / (ms / 1e3) / 1e12 / peak, 4)}
            line["e2e"] = e2e_run(model_dir, args.dtype, args.batch, args.steps)
            line["e2e"]["value"] = round(line["e2e"]["value"], 1)
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
