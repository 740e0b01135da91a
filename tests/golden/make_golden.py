#!/usr/bin/env python3
"""Makes tests/golden/gpt2_ref_*.npz: logits of the reference's own forward pass.

What it does, on the CPU, without network:
  1. writes a tiny random GPT-2 model folder with the engine's random-weights mode;
  2. rewrites it as a 32-bit GGUF in the reference's tensor names (matrices
     transposed to [out, in]) with the `gguf` package;
  3. compiles reference_forward.cpp against a CPU build tree of the reference
     (cmake -S REFERENCE -B BUILD -G Ninja -DCMAKE_BUILD_TYPE=Release; ninja
     liyab_core liyab-compat) and runs it: the first tokens whole, the rest one
     by one;
  4. stores tokens, the model's tensors and the reference's logits in an .npz.

The reference keeps its cache in 16-bit at best (include/liyab/types.h:208-213), so
its logits differ from exact arithmetic by about 1e-4 of their scale; the test that
reads these files uses that tolerance.  The reference's gpt2 row has the tanh
GELU only and no per-layer attention factor (src/compat/architecture.cpp:81-88),
so the golden models use gelu_new and no inverse-layer scaling.  It does read a
factor on the scores for the whole model (`gpt2.attention.scale`,
architecture.cpp:975-985): gpt2_ref_c has `scale_attn_weights: false`, written as
that key with the value 1, which anchors the unscaled scores on the reference too.

Usage: make_golden.py --reference /path/to/liyab --build /path/to/its/build [--only gpt2_ref_c]
"""
from __future__ import annotations

import argparse
import glob
import os
import subprocess
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CASES = {
    # name: (config, seed, prompt length fed whole, tokens fed one by one)
    "gpt2_ref_a": (dict(n_layer=2, n_embd=32, n_head=2, n_inner=80, vocab_size=96, n_positions=48,
                        layer_norm_epsilon=1e-5, activation_function="gelu_new"), 11, 20, 6),
    "gpt2_ref_b": (dict(n_layer=3, n_embd=48, n_head=3, n_inner=64, vocab_size=61, n_positions=40,
                        layer_norm_epsilon=1e-6, activation_function="gelu_new"), 12, 9, 12),
    "gpt2_ref_c": (dict(n_layer=2, n_embd=40, n_head=5, n_inner=72, vocab_size=70, n_positions=32,
                        layer_norm_epsilon=1e-5, activation_function="gelu_new", scale_attn_weights=False), 13, 14, 8),
}


def write_gguf(path: str, cfg: dict, tensors: dict) -> None:
    import gguf
    w = gguf.GGUFWriter(path, "gpt2")
    w.add_block_count(cfg["n_layer"])
    w.add_embedding_length(cfg["n_embd"])
    w.add_feed_forward_length(cfg["n_inner"])
    w.add_head_count(cfg["n_head"])
    w.add_context_length(cfg["n_positions"])
    w.add_layer_norm_eps(cfg["layer_norm_epsilon"])
    if not cfg.get("scale_attn_weights", True):
        w.add_float32("gpt2.attention.scale", 1.0)
    names = {"wte.weight": "token_embd.weight", "wpe.weight": "position_embd.weight",
             "ln_f.weight": "output_norm.weight", "ln_f.bias": "output_norm.bias"}
    per_layer = {"ln_1": "attn_norm", "attn.c_attn": "attn_qkv", "attn.c_proj": "attn_output",
                 "ln_2": "ffn_norm", "mlp.c_fc": "ffn_up", "mlp.c_proj": "ffn_down"}
    for i in range(cfg["n_layer"]):
        for ours, theirs in per_layer.items():
            for suffix in ("weight", "bias"):
                names[f"h.{i}.{ours}.{suffix}"] = f"blk.{i}.{theirs}.{suffix}"
    for name, t in tensors.items():
        a = t.astype(np.float32)
        if a.ndim == 2 and (".c_attn." in name or ".c_proj." in name or ".c_fc." in name):
            a = np.ascontiguousarray(a.T)
        w.add_tensor(names[name], a)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--build", required=True)
    ap.add_argument("--only", action="append", help="make this case only (repeatable)")
    args = ap.parse_args()
    from liyab_b200.config import parse_config
    from liyab_b200.weights import read_tensor, safetensors_describe, write_random_model

    with tempfile.TemporaryDirectory() as tmp:
        exe = os.path.join(tmp, "reference_forward")
        objs = sorted(glob.glob(os.path.join(args.build, "CMakeFiles", "liyab_core.dir", "**", "*.o"), recursive=True))
        objs += sorted(glob.glob(os.path.join(args.build, "CMakeFiles", "liyab-compat.dir", "**", "*.o"), recursive=True))
        cmd = ["g++", "-std=c++20", "-O2", "-I", os.path.join(args.reference, "include"), "-I",
               os.path.join(args.reference, "src"), os.path.join(HERE, "reference_forward.cpp"), *objs, "-o", exe,
               "-lpthread", "-ldl"]
        subprocess.run(cmd, check=True)
        for name, (raw, seed, whole, singles) in CASES.items():
            if args.only and name not in args.only:
                continue
            raw = dict(raw, model_type="gpt2")
            cfg = parse_config(raw)
            st = os.path.join(write_random_model(os.path.join(tmp, name), raw, seed, "float32"), "model.safetensors")
            tensors = {k: read_tensor(st, k, i) for k, i in safetensors_describe(st)["tensors"].items()}
            rng = np.random.default_rng(seed)
            tokens = rng.integers(0, cfg["vocab_size"], size=whole + singles).astype(np.int32)
            gguf_path = os.path.join(tmp, name + ".gguf")
            out_path = os.path.join(tmp, name + ".f32")
            write_gguf(gguf_path, raw, tensors)
            subprocess.run([exe, gguf_path, out_path, str(whole), *[str(t) for t in tokens]], check=True)
            logits = np.fromfile(out_path, dtype="<f4").reshape(len(tokens), cfg["vocab_size"])
            np.savez_compressed(os.path.join(HERE, name + ".npz"), tokens=tokens, whole=np.int32(whole),
                                logits=logits, config_json=np.bytes_(__import__("json").dumps(cfg)),
                                **{"tensor:" + k: v for k, v in tensors.items()})
            print(f"{name}: {logits.shape} logits, max |logit| {np.abs(logits).max():.4f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
