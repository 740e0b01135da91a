"""Small, self-timed workloads of single kernels and single steps, for profiling.

    python -m liyab_b200.kernel_cases gemm --m 2048 --n 768 --k 3072 --out float32 --reps 20
    python -m liyab_b200.kernel_cases decode-attention --batch 64 --context 768 --reps 20
    python -m liyab_b200.kernel_cases prefill-attention --seqs 2 --length 1024 --reps 20
    python -m liyab_b200.kernel_cases sample --rows 8 --vocab 50257 --temp 0.8 --top-k 40 --top-p 0.95
    python -m liyab_b200.kernel_cases decode-step --batch 8 --layers 12 --reps 20 [--eager]
    python -m liyab_b200.kernel_cases prefill-step --tokens 2048 --layers 12 --reps 3

Each prints one line with the CUDA-event time per repetition and the achieved rate.  The cases are what the
ncu summaries under profiles/ were captured on (one kernel, a few launches, inputs of a few hundred MB at most).
"""
from __future__ import annotations

import argparse
import os
import sys
import tempfile
import numpy as np
import torch

GPT2_SMALL = dict(model_type="gpt2", n_layer=12, n_embd=768, n_head=12, n_inner=3072, vocab_size=50257,
                  n_positions=1024, layer_norm_epsilon=1e-5, activation_function="gelu_new")
GPT2_SIZES = {"small": GPT2_SMALL,
              "medium": dict(GPT2_SMALL, n_layer=24, n_embd=1024, n_head=16, n_inner=4096),
              "large": dict(GPT2_SMALL, n_layer=36, n_embd=1280, n_head=20, n_inner=5120),
              "xl": dict(GPT2_SMALL, n_layer=48, n_embd=1600, n_head=25, n_inner=6400)}


def _timed(fn, reps: int, warmup: int = 2) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        fn()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


def _graph_timed(launch, reps: int, per_graph: int = 20) -> float:
    """Time per launch with `per_graph` launches captured in one CUDA graph: the kernel without the host's launch cost."""
    launch()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(per_graph):
            launch()
    return _timed(graph.replay, max(1, reps // per_graph)) / per_graph


class _Scratch:
    """The scratch buffers that ops.linear asks a workspace for (split-K partial sums and counters)."""

    def __init__(self, dev):
        self.dev, self.bufs = dev, {}

    def flat(self, name, n, dtype, zero=False):
        key = (name, dtype)
        if key not in self.bufs or self.bufs[key].numel() < n:
            self.bufs[key] = torch.zeros(n, dtype=dtype, device=self.dev)
        return self.bufs[key][:n]


def case_gemm(args) -> None:
    from . import ops
    dev = torch.device("cuda:0")
    odt = torch.float32 if args.out == "float32" else torch.bfloat16
    a = torch.randn(args.m, args.k, device=dev).to(torch.bfloat16)
    w = (torch.randn(args.n, args.k, device=dev) * 0.05).to(torch.bfloat16)
    bias = torch.randn(args.n, device=dev)
    out = torch.zeros(args.m, args.n, dtype=odt, device=dev)
    res = out if odt == torch.float32 else None
    if args.weights > 1:
        # A chain of the same product over several weight matrices (more bytes than L2 holds: every launch streams
        # its weights from DRAM, as a layer's products do in a step).
        ws, many, turn = _Scratch(dev), [w] + [w.clone() for _ in range(args.weights - 1)], [0]

        def launch():
            wi = many[turn[0] % len(many)]
            turn[0] += 1
            if args.rows:
                ops.gemm_rows(a, wi, bias, out, args.m, args.act, residual=res)
            else:
                ops.linear(a, wi, bias, out, args.m, args.act, residual=res, workspace=ws)
    elif args.rows:
        launch = lambda: ops.gemm_rows(a, w, bias, out, args.m, args.act, residual=res)
    elif args.one_tile:
        launch = lambda: ops.gemm_tcgen05(a, w, bias, out, args.m, args.act, residual=res, token_tile=args.tile)
    elif args.m > 64 and ops.gemm_persistent_tile(a, w, out, args.m, res) > 0:
        launch = lambda: ops.gemm_persistent(a, w, bias, out, args.m, args.act, residual=res, feature_tile=args.tile)
    else:
        ws = _Scratch(dev)
        launch = lambda: ops.linear(a, w, bias, out, args.m, args.act, residual=res, workspace=ws)
    ms = _graph_timed(launch, args.reps) if args.graph else _timed(launch, args.reps)
    print(f"gemm M={args.m} N={args.n} K={args.k} out={args.out}: {ms * 1e3:.1f} us per launch (includes the host's "
          f"launch cost when the kernel is shorter), {2 * args.m * args.n * args.k / ms / 1e9:.1f} TFLOP/s, "
          f"{(args.n * args.k * 2) / ms / 1e6:.1f} GB/s of weights, status {ops.device_status()}")


def case_decode_attention(args) -> None:
    from . import ops
    dev = torch.device("cuda:0")
    B, H, hd, ps, ctx = args.batch, args.heads, args.head_dim, 16, args.context
    pages_per = -(-ctx // ps)
    cache = torch.randn(B * pages_per, 2, H, ps, hd, device=dev).to(torch.bfloat16)
    table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
    q = torch.randn(B, H * hd, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    positions = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    tensor = ops.decode_attention_kernels(H, H, hd, ps)[1] and not args.scalar
    splits = args.splits or ops.decode_splits(B, H, ctx, tensor_cores=tensor)
    partial = torch.empty(B * H * splits * (hd + 2), device=dev)
    counters = torch.zeros(B * H, dtype=torch.int32, device=dev)
    def launch():
        ops.decode_attention(q, cache, positions, table, out, partial, counters, B, H, H, hd, ps, hd ** -0.5, 0, splits,
                             tensor_cores=tensor)

    ms = _graph_timed(launch, args.reps) if args.graph else _timed(launch, args.reps)
    nbytes = B * ctx * 2 * H * hd * 2
    kind = "tensor-core" if tensor else "scalar"
    print(f"decode-attention ({kind}) batch={B} heads={H} head_dim={hd} context={ctx} splits={splits}: {ms * 1e3:.1f} us, "
          f"{nbytes / ms / 1e6:.1f} GB/s of cache ({nbytes / 1e6:.1f} MB)")


def case_generic_attention(args) -> None:
    """The 32-bit engine's attention: `batch` requests at `context`, each with `new` tokens in this step."""
    from . import ops
    dev = torch.device("cuda:0")
    dt = torch.float32 if args.dtype == "float32" else torch.bfloat16
    B, H, hd, ps, ctx, new = args.batch, args.heads, args.head_dim, 16, args.context, args.new
    pages_per = -(-ctx // ps)
    cache = torch.randn(B * pages_per, 2, H, ps, hd, device=dev).to(dt)
    table = torch.arange(B * pages_per, dtype=torch.int32, device=dev).view(B, pages_per)
    q = torch.randn(B * new, H * hd, device=dev).to(dt)
    out = torch.empty_like(q)
    tok_seq = torch.arange(B, dtype=torch.int32, device=dev).repeat_interleave(new)
    positions = torch.arange(ctx - new, ctx, dtype=torch.int32, device=dev).repeat(B)
    launch = lambda: ops.paged_attention_generic(q, cache, tok_seq, positions, table, out, B * new, H, H, hd, ps, hd ** -0.5, 0)
    ms = _graph_timed(launch, args.reps) if args.graph else _timed(launch, args.reps)
    nbytes = B * ctx * 2 * H * hd * cache.element_size()
    print(f"generic-attention {args.dtype} batch={B} new={new} heads={H} head_dim={hd} context={ctx}: {ms * 1e3:.1f} us, "
          f"{nbytes / ms / 1e6:.1f} GB/s of cache ({nbytes / 1e6:.1f} MB)")


def case_gemm_f32(args) -> None:
    """The 32-bit engine's product (FMA pipe, one summation order for every number of tokens)."""
    from . import ops
    dev = torch.device("cuda:0")
    a = torch.randn(args.m, args.k, device=dev)
    w = torch.randn(args.n, args.k, device=dev) * 0.05
    bias = torch.randn(args.n, device=dev)
    out = torch.zeros(args.m, args.n, device=dev)
    launch = lambda: ops.gemm_ffma(a, w, bias, out, args.m, args.act)
    ms = _graph_timed(launch, args.reps) if args.graph else _timed(launch, args.reps)
    print(f"gemm-f32 M={args.m} N={args.n} K={args.k}: {ms * 1e3:.1f} us per launch, {2 * args.m * args.n * args.k / ms / 1e9:.2f} TFLOP/s, "
          f"{(args.n * args.k * 4) / ms / 1e6:.1f} GB/s of weights")


def case_prefill_attention(args) -> None:
    from . import ops
    dev = torch.device("cuda:0")
    S, L, H, hd, ps = args.seqs, args.length, args.heads, args.head_dim, 16
    pages_per = -(-L // ps)
    cache = torch.randn(S * pages_per, 2, H, ps, hd, device=dev).to(torch.bfloat16)
    table = torch.arange(S * pages_per, dtype=torch.int32, device=dev).view(S, pages_per)
    q = torch.randn(S * L, H * hd, device=dev).to(torch.bfloat16)
    out = torch.empty_like(q)
    q_start = torch.arange(0, (S + 1) * L, L, dtype=torch.int32, device=dev)
    n_past = torch.zeros(S, dtype=torch.int32, device=dev)

    def launch():
        ops.prefill_attention(q, cache, q_start, n_past, table, out, S, L, H, H, hd, ps, hd ** -0.5, 0,
                              tcgen05=False if args.mma_sync else None)

    ms = _graph_timed(launch, args.reps) if args.graph else _timed(launch, args.reps)
    flop = S * H * (L * L / 2) * hd * 4
    print(f"prefill-attention seqs={S} length={L} heads={H} head_dim={hd}: {ms * 1e3:.1f} us, {flop / ms / 1e9:.1f} TFLOP/s "
          f"(causal half of the square)")


def case_sample(args) -> None:
    from . import ops
    dev = torch.device("cuda:0")
    R, V = args.rows, args.vocab
    logits = torch.randn(R, V, device=dev) * args.spread
    temp = torch.full((R,), args.temp, device=dev)
    top_k = torch.full((R,), args.top_k, dtype=torch.int32, device=dev)
    top_p = torch.full((R,), args.top_p, device=dev)
    u = torch.rand(R, dtype=torch.float64, device=dev)
    ids = torch.empty(R, dtype=torch.int32, device=dev)
    ms = _graph_timed(lambda: ops.sample(logits, R, temp, top_k, top_p, u, ids), args.reps)
    print(f"sample rows={R} vocab={V} temp={args.temp} top_k={args.top_k} top_p={args.top_p}: {ms * 1e3:.1f} us "
          f"(20 launches per CUDA graph)")


def _model_folder(layers: int, dtype: str, size: str = "small") -> str:
    """A random model of the asked size in a temporary folder that is removed when the process ends."""
    import atexit
    import shutil
    from .weights import write_random_model
    tmp = tempfile.mkdtemp(prefix="liyab_b200_case_")
    atexit.register(shutil.rmtree, tmp, ignore_errors=True)
    return write_random_model(os.path.join(tmp, "m"), dict(GPT2_SIZES[size], n_layer=layers or GPT2_SIZES[size]["n_layer"]), 0, dtype)


def case_decode_step(args) -> None:
    """A few decode steps of the whole model through the library's own measurement (what bench.py times)."""
    from .engine import Replayer
    B = args.batch
    rep = Replayer(_model_folder(args.layers, args.dtype, args.size), args.dtype, max_tokens=B * 1024, max_requests=B,
                   cuda_graphs=not args.eager, fused_decode=args.fused and not args.no_fused, max_step_tokens=1024)
    r = rep.bench_decode(B, args.context, args.reps, 3)
    path = "fused" if r["fused_steps"] else ("graph" if r["graph_steps"] else "parts")
    print(f"decode-step size={args.size} batch={B} layers={len(rep.info['spec']['layers'])} context~{r['mean_context']:.0f} path={path}: "
          f"{r['ms_per_step'] * 1e3:.1f} us per step, {B / r['ms_per_step'] * 1e3:.0f} tokens/s, {r['kernel_launches'] // args.reps} launches a step")
    if args.stamps and r["fused_steps"]:
        # Where the one-kernel step's time goes: the five barriers of layer 5 (numbers 27..31), all blocks' arrivals.
        rep.set("fused_stamps", 1)
        rep.bench_decode(B, args.context, 3, 1)
        t = rep.fused_stamps().astype(np.float64) / 1e3
        n_blocks = int(np.count_nonzero(t[256:256 + 160]))
        last_barrier = int(np.flatnonzero(t[:126]).max())
        print(f"  whole kernel after its first barrier: {t[last_barrier] - t[1]:.1f} us over {last_barrier - 1} barriers; head {t[127] - t[126]:.1f} us; "
              f"from block 0's start to the first barrier's end {t[1] - t[0]:.1f} us")
        names = ["LayerNorm + projection", "attention", "output projection", "LayerNorm + up", "down"]
        for j, name in enumerate(names):
            arrive = np.sort(t[256 + 160 * j:256 + 160 * j + n_blocks])
            before, after = t[26 + j], t[27 + j]
            print(f"  layer 5 {name:>22}: work {arrive[0] - before:5.2f} / {np.median(arrive) - before:5.2f} / {arrive[-1] - before:5.2f} us "
                  f"(first / median / last block to arrive), barrier left {after - arrive[-1]:5.2f} us after the last arrival, phase {after - before:5.2f} us")


def case_prefill_step(args) -> None:
    from .engine import Replayer
    n_seq = max(1, args.tokens // 1024)
    per = args.tokens // n_seq
    rep = Replayer(_model_folder(args.layers, args.dtype, args.size), args.dtype, max_tokens=2 * args.tokens,
                   cuda_graphs=not args.eager, max_step_tokens=args.tokens)
    r = rep.bench_prefill(n_seq, per, args.reps)
    print(f"prefill-step size={args.size} tokens={n_seq}x{per} layers={len(rep.info['spec']['layers'])}: best {r['ms_per_step']:.3f} ms, "
          f"median {r['wall_ms_per_step']:.3f} ms per step, {n_seq * per / r['ms_per_step'] * 1e3:.0f} tokens/s, {r['kernel_launches']} launches")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m liyab_b200.kernel_cases")
    sub = ap.add_subparsers(dest="case", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=2048)
    g.add_argument("--n", type=int, default=768)
    g.add_argument("--k", type=int, default=3072)
    g.add_argument("--out", default="bfloat16", choices=["bfloat16", "float32"])
    g.add_argument("--act", default="none", choices=["none", "gelu_tanh", "gelu_erf"])
    g.add_argument("--tile", type=int, default=0, help="feature tile of the persistent kernel (token tile with --one-tile)")
    g.add_argument("--graph", action="store_true", help="time 20 launches captured in a CUDA graph")
    g.add_argument("--one-tile", action="store_true", help="the one-tile-per-block kernel also for many tokens")
    g.add_argument("--weights", type=int, default=1, help="cycle through this many copies of the weights (with --graph: 20 per graph)")
    g.add_argument("--rows", action="store_true", help="the one-launch mma.sync product (up to 64 tokens) whatever the size")
    g.add_argument("--reps", type=int, default=20)
    d = sub.add_parser("decode-attention")
    d.add_argument("--batch", type=int, default=64)
    d.add_argument("--heads", type=int, default=12)
    d.add_argument("--head-dim", type=int, default=64)
    d.add_argument("--context", type=int, default=768)
    d.add_argument("--reps", type=int, default=20)
    d.add_argument("--splits", type=int, default=0, help="key ranges per request and head (0: the engine's choice)")
    d.add_argument("--graph", action="store_true", help="time 20 launches captured in a CUDA graph")
    d.add_argument("--scalar", action="store_true", help="the scalar kernel even where the tensor-core one takes the shape")
    ga = sub.add_parser("generic-attention")
    ga.add_argument("--batch", type=int, default=8)
    ga.add_argument("--new", type=int, default=1, help="tokens of each request in this step")
    ga.add_argument("--heads", type=int, default=12)
    ga.add_argument("--head-dim", type=int, default=64)
    ga.add_argument("--context", type=int, default=768)
    ga.add_argument("--dtype", default="float32", choices=["bfloat16", "float32"])
    ga.add_argument("--reps", type=int, default=20)
    ga.add_argument("--graph", action="store_true", help="time 20 launches captured in a CUDA graph")
    gf = sub.add_parser("gemm-f32")
    gf.add_argument("--m", type=int, default=8)
    gf.add_argument("--n", type=int, default=2304)
    gf.add_argument("--k", type=int, default=768)
    gf.add_argument("--act", default="none", choices=["none", "gelu_tanh", "gelu_erf"])
    gf.add_argument("--reps", type=int, default=20)
    gf.add_argument("--graph", action="store_true", help="time 20 launches captured in a CUDA graph")
    a = sub.add_parser("prefill-attention")
    a.add_argument("--seqs", type=int, default=2)
    a.add_argument("--length", type=int, default=1024)
    a.add_argument("--heads", type=int, default=12)
    a.add_argument("--head-dim", type=int, default=64)
    a.add_argument("--reps", type=int, default=20)
    a.add_argument("--graph", action="store_true", help="time 20 launches captured in a CUDA graph")
    a.add_argument("--mma-sync", action="store_true", help="the mma.sync kernel even where the tcgen05 one takes the shape")
    sm = sub.add_parser("sample")
    sm.add_argument("--rows", type=int, default=8)
    sm.add_argument("--vocab", type=int, default=50257)
    sm.add_argument("--temp", type=float, default=0.8)
    sm.add_argument("--top-k", type=int, default=40)
    sm.add_argument("--top-p", type=float, default=0.95)
    sm.add_argument("--spread", type=float, default=3.0, help="standard deviation of the random logits (8: peaked like a model's)")
    sm.add_argument("--reps", type=int, default=400)
    for name in ("decode-step", "prefill-step"):
        p = sub.add_parser(name)
        p.add_argument("--batch", type=int, default=8)
        p.add_argument("--tokens", type=int, default=2048)
        p.add_argument("--context", type=int, default=512)
        p.add_argument("--layers", type=int, default=0, help="fewer layers than the size has (0: all)")
        p.add_argument("--size", default="small", choices=sorted(GPT2_SIZES))
        p.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
        p.add_argument("--reps", type=int, default=10)
        p.add_argument("--eager", action="store_true", help="no captured graphs")
        p.add_argument("--no-fused", action="store_true", help="not the one-kernel decode step")
        p.add_argument("--fused", action="store_true", help="decode steps of up to 16 requests as one persistent kernel (default: part by part)")
        p.add_argument("--stamps", action="store_true", help="decode-step: per-phase times from inside the one-kernel step")
    args = ap.parse_args(argv)
    {"gemm": case_gemm, "generic-attention": case_generic_attention, "gemm-f32": case_gemm_f32, "decode-attention": case_decode_attention, "prefill-attention": case_prefill_attention, "sample": case_sample, "decode-step": case_decode_step,
     "prefill-step": case_prefill_step}[args.case](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
