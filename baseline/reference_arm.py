"""The reference arm of bench.py: the unmodified reference, through its own tools, for the benchmark's metric.

liyab is a CMake C++ project without a Python package (pip finds neither setup.py nor pyproject.toml), so it is
configured and built with cmake into baseline/_ref/build, which is not part of the repository's history:

    cmake -S <reference> -B baseline/_ref/build -G Ninja -DCMAKE_BUILD_TYPE=Release
    ninja -C baseline/_ref/build liyab-bench liyab-seq-bench liyab-cli

It is a CPU engine (its GPU paths are Metal and Vulkan), so the arm runs on this machine's CPU cores.  The model is
GPT-2 small with random weights (the same seed and init as the engine's arm), written as a 16-bit GGUF in the
reference's tensor names, with a byte-level token table so that the reference's public API, which has no entry for
token ids without a tokenizer, accepts it.  Prefill: `liyab-bench --prefill` (synthetic token ids, its own
measurement).  Decode: `liyab-seq-bench --sequences B` (B sequences decoding at once through Engine::open_sequence,
its own measurement and its own prompts).
"""
from __future__ import annotations

import json
import os
import re
import shutil
import subprocess
import sys
import tempfile
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
BUILD = os.path.join(HERE, "_ref", "build")
REFERENCE = os.environ.get("LIYAB_REFERENCE", "/root/reference")
TOOLS = ("liyab-bench", "liyab-seq-bench")


def unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def ensure_built() -> str:
    """Empty when the tools are there (built now if they can be), else the reason they are not."""
    if all(os.path.isfile(os.path.join(BUILD, t)) for t in TOOLS):
        return ""
    if not os.path.isdir(REFERENCE):
        return f"baseline/_ref/build holds no built reference and its source tree {REFERENCE} is absent"
    for tool in ("cmake", "ninja", "g++"):
        if shutil.which(tool) is None:
            return f"baseline/_ref/build holds no built reference and {tool} is not installed to build it"
    os.makedirs(BUILD, exist_ok=True)
    for cmd in (["cmake", "-S", REFERENCE, "-B", BUILD, "-G", "Ninja", "-DCMAKE_BUILD_TYPE=Release"], ["ninja", "-C", BUILD, *TOOLS]):
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        if proc.returncode != 0:
            return f"building the reference failed at `{' '.join(cmd[:2])}`: {proc.stdout.strip().splitlines()[-1][:200] if proc.stdout.strip() else 'no output'}"
    return ""


def byte_level_tokens(vocab: int):
    """GPT-2's byte-to-character table for the first 256 ids, filler names for the rest: every text then encodes to
    its bytes, one token each."""
    keep = list(range(ord("!"), ord("~") + 1)) + list(range(0xA1, 0xAD)) + list(range(0xAE, 0x100))
    chars, extra = {}, 0
    for b in range(256):
        if b in keep:
            chars[b] = chr(b)
        else:
            chars[b] = chr(256 + extra)
            extra += 1
    # one merge ("a a" -> "aa", id 256) so that the table is a valid BPE vocabulary
    return [chars[b] for b in range(256)] + ["aa"] + [f"<filler_{i}>" for i in range(257, vocab)]


def write_gguf(path: str, cfg: dict, folder: str) -> None:
    """The engine's random-weights folder rewritten in the reference's names, matrices [out, in], 16-bit floats."""
    import gguf
    import numpy as np
    from liyab_b200.weights import read_tensor, safetensors_describe
    w = gguf.GGUFWriter(path, "gpt2")
    w.add_block_count(cfg["n_layer"])
    w.add_embedding_length(cfg["n_embd"])
    w.add_feed_forward_length(cfg["n_inner"])
    w.add_head_count(cfg["n_head"])
    w.add_context_length(cfg["n_positions"])
    w.add_layer_norm_eps(cfg["layer_norm_epsilon"])
    w.add_tokenizer_model("gpt2")
    w.add_token_list(byte_level_tokens(cfg["vocab_size"]))
    w.add_token_merges(["a a"])
    w.add_token_types([1] * cfg["vocab_size"])
    w.add_eos_token_id(cfg["vocab_size"] - 1)
    names = {"wte.weight": "token_embd.weight", "wpe.weight": "position_embd.weight",
             "ln_f.weight": "output_norm.weight", "ln_f.bias": "output_norm.bias"}
    per_layer = {"ln_1": "attn_norm", "attn.c_attn": "attn_qkv", "attn.c_proj": "attn_output",
                 "ln_2": "ffn_norm", "mlp.c_fc": "ffn_up", "mlp.c_proj": "ffn_down"}
    for i in range(cfg["n_layer"]):
        for ours, theirs in per_layer.items():
            for suffix in ("weight", "bias"):
                names[f"h.{i}.{ours}.{suffix}"] = f"blk.{i}.{theirs}.{suffix}"
    st = os.path.join(folder, "model.safetensors")
    for name, info in safetensors_describe(st)["tensors"].items():
        a = read_tensor(st, name, info).astype(np.float32)
        if a.ndim == 2 and (".c_attn." in name or ".c_proj." in name or ".c_fc." in name):
            a = np.ascontiguousarray(a.T)
        w.add_tensor(names[name], a.astype(np.float16) if a.ndim == 2 else a)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def run(args) -> int:
    why = ensure_built()
    if why:
        return unavailable(why)
    try:
        import gguf  # noqa: F401
    except ImportError:
        return unavailable("the python package gguf (to write the model file the reference reads) is not installed")
    sys.path.insert(0, ROOT)
    from bench import PREFILL_TOKENS, SIZES
    from liyab_b200.weights import write_random_model
    cfg = SIZES[args.size]
    batch = min(args.batch, 4)          # liyab-seq-bench has four tasks: "1 to 4 sequences (one task each)"
    n_new = max(8, min(args.steps, 64))
    env = dict(os.environ, LD_LIBRARY_PATH=BUILD + os.pathsep + os.environ.get("LD_LIBRARY_PATH", ""))
    with tempfile.TemporaryDirectory(prefix="liyab_ref_") as tmp:
        folder = write_random_model(os.path.join(tmp, "m"), cfg, 0, "float32")
        model = os.path.join(tmp, "gpt2.gguf")
        write_gguf(model, cfg, folder)
        t0 = time.perf_counter()
        pre = subprocess.run([os.path.join(BUILD, "liyab-bench"), "--prefill", model, "--tokens", str(PREFILL_TOKENS // 2), "--batch", "512",
                              "--kv", "f16", "--repeat", "2"], capture_output=True, text=True, env=env, timeout=1500)
        dec = subprocess.run([os.path.join(BUILD, "liyab-seq-bench"), "-m", model, "--sequences", str(batch), "-n", str(n_new), "--kv", "f16",
                              "--backend", "cpu"], capture_output=True, text=True, env=env, timeout=1500)
        seconds = time.perf_counter() - t0
    text = pre.stdout + "\n" + dec.stdout
    if pre.returncode != 0 or dec.returncode != 0:
        tail = (pre.stderr + dec.stderr).strip().splitlines()
        return unavailable(f"the reference's tools failed on the random GPT-2 model: {tail[-1][:300] if tail else 'no message'}")
    prefill = [float(x) for x in re.findall(r"([0-9.]+)\s*tok/s", pre.stdout)]
    # its table: seqs, seq tok/s, slowest, together, in turns, gain, same, scheduler
    row = next((l.split() for l in reversed(dec.stdout.splitlines()) if l.split()[:1] == [str(batch)]), None)
    if row is None or len(row) < 7:
        return unavailable("liyab-seq-bench printed no row for %d sequences: %s" % (batch, dec.stdout.strip()[-200:]))
    value, in_turns, same = float(row[3]), float(row[4]), row[6]
    line = {"impl": "reference", "metric": f"GPT-2 {args.size} decode tokens/s (batch {batch}, 512-token prompts, contexts 512-1024)",
            "value": round(value, 2), "unit": "tokens/s", "n_gpus": 1, "steps": n_new, "warmup": 1, "ms_per_step": round(batch / value * 1e3, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "fp16 weights, f16 cache, fp32 activations (the reference has no bf16 engine mode)",
            "data": "synthetic: random-init weights (seed 0); liyab-seq-bench's own writing prompts, byte-level token table",
            "config": {"model": f"gpt2-{args.size}", "n_layer": cfg["n_layer"], "n_embd": cfg["n_embd"], "n_head": cfg["n_head"], "n_inner": cfg["n_inner"],
                       "vocab_size": cfg["vocab_size"], "n_positions": cfg["n_positions"], "global_batch": batch, "asked_batch": args.batch,
                       "batch_note": "the reference's stock tool decodes at most 4 sequences together", "device": "CPU (the reference has no CUDA path)",
                       "tool": "liyab-seq-bench --sequences B (together), liyab-bench --prefill", "in_turns_tokens_per_s": in_turns,
                       "same": same, "seconds": round(seconds, 1)},
            "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "the tool's own end-to-end figure through the reference's public API; no device copies on a CPU engine"},
            "gpu_launches": 0}
    if prefill:
        line["prefill"] = {"value": max(prefill), "tokens": PREFILL_TOKENS // 2, "note": "liyab-bench --prefill, best of 2"}
    line["tool_output_tail"] = text.strip()[-600:]
    print(json.dumps(line))
    return 0
