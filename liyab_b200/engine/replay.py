"""Trace replay: given token ids go through the model step by step and the
logits at the wanted places are written out.  Nothing is sampled.

It drives the framework's own model, step function, cache manager and kernels:
the ones that generation uses.  The reference's counterparts are its schedule
harness (Plan / Trace / run_batched: tests/test_sequences.cpp:87-252) and the
teacher-forced passes of liyab-kl (tools/liyab_kl.cpp:45-47).

Input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, OUT/<step>.f32 receives the logits at
the wanted places, in the order of the entries and of `want`, as little-endian
float32 [wanted, vocab].  After every step a line `done <step>` is printed.
"""
from __future__ import annotations

import json
import os
import sys
from typing import IO, Optional

import numpy as np
import torch

from ..cache.pages import CacheManager
from ..models.loading import load_model
from ..status import LiyabError
from .step import StepEntry, Stepper

REPLAY_PAGE_SIZE = 16
MAX_LIVE_REQUESTS = 16


def build_replayer(model_dir: str, dtype: str, max_tokens: int, device: str = "cuda:0",
                   page_size: int = REPLAY_PAGE_SIZE, max_requests: int = MAX_LIVE_REQUESTS, fused_decode: bool = True):
    model, _ = load_model(model_dir, dtype, device)
    num_pages = max(1, (max_tokens + page_size - 1) // page_size)
    cache = CacheManager(model.kv_needs(), model.state_needs(), page_size, num_pages, max_requests,
                         dtype=model.runtime.dtype, device=model.runtime.device)
    return model, cache, Stepper(model, cache, fused_decode=fused_decode)


def replay(model_dir: str, dtype: str, out_dir: str, max_tokens: int, lines: IO[str], done: Optional[IO[str]] = None,
           device: str = "cuda:0", page_size: int = REPLAY_PAGE_SIZE) -> int:
    os.makedirs(out_dir, exist_ok=True)
    done = done or sys.stdout
    _, cache, stepper = build_replayer(model_dir, dtype, max_tokens, device, page_size)
    for line in lines:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step_id = record["step"]
        entries = []
        for e in record.get("entries", []):
            if not cache.is_open(e["id"]):
                cache.open(e["id"])
            entries.append(StepEntry(request=e["id"], tokens=[int(t) for t in e["tokens"]],
                                     want=[int(w) for w in e.get("want", [])]))
        if entries:
            out = stepper.step(entries)
            if out.logits is not None and out.logits.shape[0] > 0:
                data = out.logits.detach().to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                tmp = os.path.join(out_dir, f".{step_id}.f32.tmp")
                data.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step_id}.f32"))
        for rid in record.get("end", []):
            if cache.is_open(rid):
                cache.close(rid)
        print(f"done {step_id}", file=done, flush=True)
    return 0


def main(argv=None) -> int:
    import argparse
    ap = argparse.ArgumentParser(prog="trace_run", description="Replay given token ids through the engine and write logits.")
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder that receives <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (each rounded up to 64)")
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--page-size", type=int, default=REPLAY_PAGE_SIZE, choices=[16, 32, 64])
    args = ap.parse_args(argv)
    try:
        return replay(args.model, args.dtype, args.out, args.max_tokens, sys.stdin, sys.stdout, args.device,
                      args.page_size)
    except LiyabError as e:
        print(f"trace_run: {e}", file=sys.stderr, flush=True)
        return 1
