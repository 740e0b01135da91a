"""The command line, in the manner of the reference's liyab-cli.

Options keep the reference's names and meanings where it has them
(tools/liyab_cli.cpp:242-334: -m, -p, -n, --temp, --top-k, --top-p, --seed, --ctx,
--json, --tokenize, --then) with their defaults (-n 128, --temp 0.8, --top-k 40,
--top-p 0.95, random seed).  The engine has no tokenizer, so a prompt is a list
of token ids ("-p 464,3290,318") or `--prompt-len N` random ids; `--kv` becomes
`--dtype` (the cache has the compute type).  The summary on stderr and the JSON
lines follow tools/liyab_cli.cpp:145-240.
"""
from __future__ import annotations

import argparse
import json
import sys
import tempfile
import time
from typing import List

import numpy as np

from .status import LiyabError


def _ids(text: str) -> List[int]:
    try:
        return [int(t) for t in text.replace(" ", ",").split(",") if t != ""]
    except ValueError:
        raise argparse.ArgumentTypeError(f"a prompt is a list of token ids, e.g. 464,3290,318 (got {text!r})")


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="liyab-cli", description="Generate token ids with the liyab_b200 engine.")
    ap.add_argument("-m", "--model", help="model folder (config.json + model.safetensors)")
    ap.add_argument("--random-weights", metavar="CONFIG.json",
                    help="no model folder: write one with random weights from this configuration first")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of --random-weights (default 0)")
    ap.add_argument("-p", "--prompt", type=_ids, action="append", help="prompt token ids, comma separated (repeatable)")
    ap.add_argument("--prompt-len", type=int, default=0, help="instead of -p: this many uniform random token ids")
    ap.add_argument("--prompt-seed", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1, help="with --prompt-len: this many prompts served together")
    ap.add_argument("--tokenize", action="store_true", help="print the prompt's token ids and exit")
    ap.add_argument("-n", type=int, default=128, dest="max_tokens", help="max new tokens (default 128), per turn")
    ap.add_argument("--then", type=_ids, action="append", default=[],
                    help="a follow-up turn (repeatable): its prompt is the previous prompt, the reply and these ids")
    ap.add_argument("--json", action="store_true", help="stdout: one JSON line after loading and one per turn")
    ap.add_argument("--temp", type=float, default=0.8, help="temperature, 0 = greedy (default 0.8)")
    ap.add_argument("--top-k", type=int, default=40, help="(default 40)")
    ap.add_argument("--top-p", type=float, default=0.95, help="(default 0.95)")
    ap.add_argument("--seed", type=int, default=0, help="RNG seed (default random)")
    ap.add_argument("--ignore-eos", action="store_true", help="do not stop at the end-of-sequence token")
    ap.add_argument("--ctx", type=int, default=0, help="context length (default: the model's)")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32", "bf16", "fp32"],
                    help="compute and cache type (default bfloat16)")
    ap.add_argument("--max-batched-tokens", type=int, default=2048, help="token budget of one step")
    ap.add_argument("--max-requests", type=int, default=64)
    ap.add_argument("--page-size", type=int, default=16, choices=[16, 32, 64])
    ap.add_argument("--num-pages", type=int, default=0, help="cache pages (default: sized from free memory)")
    ap.add_argument("--no-graphs", action="store_true", help="do not replay captured CUDA graphs for decode steps")
    return ap


def _print_stats(stats, out=sys.stderr) -> None:
    print("\n=== Generation ===\n"
          f"prompt: {stats.prompt_tokens} tokens (0 reused), {stats.prefill_ms:.1f} ms, TTFT {stats.ttft_ms:.1f} ms\n"
          f"decode: {stats.generated_tokens} tokens, {stats.decode_ms:.1f} ms, {stats.tokens_per_second:.2f} tok/s"
          f"{', cancelled' if stats.cancelled else ''}\n"
          f"memory: KV {stats.kv_cache_bytes / 2**20:.1f} MiB", file=out)


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    try:
        return _run(args)
    except LiyabError as e:
        print(f"liyab-cli: {e}", file=sys.stderr)
        return 1


def _run(args) -> int:
    from .config import parse_config
    from .sampling.params import SamplingParams
    tmp = None
    model = args.model
    if args.random_weights:
        from .weights import write_random_model
        with open(args.random_weights, "r", encoding="utf-8") as f:
            cfg = parse_config(json.load(f))
        tmp = tempfile.TemporaryDirectory(prefix="liyab_b200_model_")
        model = write_random_model(tmp.name, cfg, args.weights_seed, "bfloat16" if args.dtype in ("bfloat16", "bf16") else "float32")
    if not model:
        print("liyab-cli: -m MODEL (or --random-weights CONFIG.json) is required", file=sys.stderr)
        return 2
    prompts: List[List[int]] = list(args.prompt or [])
    if args.prompt_len > 0:
        from .config import read_config
        vocab = read_config(model).model_spec().vocab_size
        rng = np.random.default_rng(args.prompt_seed)
        prompts += [rng.integers(0, vocab, size=args.prompt_len).astype(int).tolist() for _ in range(max(1, args.batch))]
    if not prompts:
        print("liyab-cli: a prompt is required (-p IDS or --prompt-len N)", file=sys.stderr)
        return 2
    if args.tokenize:
        for p in prompts:
            print(" ".join(str(t) for t in p))
        return 0
    from .engine.engine import Engine, EngineConfig
    t0 = time.perf_counter()
    engine = Engine(EngineConfig(model=model, dtype=args.dtype, context_length=args.ctx,
                                 max_batched_tokens=args.max_batched_tokens, max_requests=args.max_requests,
                                 page_size=args.page_size, num_pages=args.num_pages, cuda_graphs=not args.no_graphs))
    if args.json:
        print(json.dumps({"load_ms": round((time.perf_counter() - t0) * 1e3, 1), "context": engine.max_positions,
                          "describe": engine.describe()}), flush=True)
    else:
        print(engine.describe(), file=sys.stderr)
    params = SamplingParams(temperature=args.temp, top_k=args.top_k, top_p=args.top_p, seed=args.seed,
                            max_tokens=args.max_tokens, ignore_eos=args.ignore_eos)
    turns = [None] + list(args.then)
    for follow in turns:
        if follow is not None:
            prompts = [p + r.tokens + follow for p, r in zip(prompts, results)]
        results = engine.generate_batch(prompts, params)
        for r in results:
            if r.error is not None:
                print(f"liyab-cli: {r.error}", file=sys.stderr)
            if args.json:
                s = r.stats
                print(json.dumps({"prompt_tokens": s.prompt_tokens, "generated_tokens": s.generated_tokens,
                                  "prefill_ms": round(s.prefill_ms, 3), "decode_ms": round(s.decode_ms, 3),
                                  "ttft_ms": round(s.ttft_ms, 3), "tokens_per_second": round(s.tokens_per_second, 2),
                                  "kv_cache_bytes": s.kv_cache_bytes, "finish_reason": r.finish_reason,
                                  "tokens": r.tokens}), flush=True)
            else:
                print(" ".join(str(t) for t in r.tokens), flush=True)
                _print_stats(r.stats)
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
