"""Builds replay traces (lists of steps) and runs them through a Stepper.

A trace is a list of steps; a step is (entries, end) with entries
[(request, tokens, want)].  `collect` returns {(request, position): logits row}.
The four shapes are the ones the engine must agree on: whole, most of it then
the last tokens one by one, portions of changing size, and several requests
mixed with so few pages that freed ones are used again.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

import numpy as np

Step = Tuple[List[Tuple[str, List[int], List[int]]], List[str]]


def whole(requests: Dict[str, List[int]]) -> List[Step]:
    return [([(r, toks, list(range(len(toks))))], [r]) for r, toks in requests.items()]


def tail_one_by_one(requests: Dict[str, List[int]], tail: int = 32) -> List[Step]:
    steps: List[Step] = []
    for r, toks in requests.items():
        head = max(len(toks) - tail, 0)
        if head:
            steps.append(([(r, toks[:head], list(range(head)))], []))
        for i in range(head, len(toks)):
            steps.append(([(r, [toks[i]], [0])], [r] if i == len(toks) - 1 else []))
    return steps


def changing_portions(requests: Dict[str, List[int]], sizes: Sequence[int] = (16, 8, 5, 3, 2, 2, 7, 2, 11, 4)) -> List[Step]:
    steps: List[Step] = []
    for r, toks in requests.items():
        at, k = 0, 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            steps.append(([(r, toks[at:at + n], list(range(n)))], [r] if at + n == len(toks) else []))
            at += n
    return steps


def mixed(requests: Dict[str, List[int]], max_live: int = 4, seed: int = 0, prompt_frac: float = 0.6,
          portion: int = 16) -> List[Step]:
    """Up to `max_live` requests at a time: each prefills in portions (some tiny), then
    goes on one token per step ("decode") beside the others' portions; late joiners
    enter when a request ends; a request now and then sits a step out."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    live: List[Dict] = []
    steps: List[Step] = []
    while waiting or live:
        while waiting and len(live) < max_live:
            r, toks = waiting.pop(0)
            live.append(dict(id=r, toks=toks, at=0, prompt=max(1, int(len(toks) * prompt_frac))))
        entries, end = [], []
        for s in live:
            if len(live) > 1 and rng.random() < 0.15:
                continue                                    # left out of this step, goes on later
            if s["at"] < s["prompt"]:
                n = min(int(rng.choice([2, 3, portion, portion, 5])), s["prompt"] - s["at"])
            else:
                n = 1
            n = min(n, len(s["toks"]) - s["at"])
            entries.append((s["id"], s["toks"][s["at"]:s["at"] + n], list(range(n))))
            s["at"] += n
            if s["at"] == len(s["toks"]):
                end.append(s["id"])
        live = [s for s in live if s["id"] not in end]
        if entries:
            steps.append((entries, end))
    return steps


def peak_tokens(steps: List[Step], round_to: int = 64) -> int:
    """The most tokens live requests hold at any time, each rounded up to `round_to`."""
    held: Dict[str, int] = {}
    peak = 0
    for entries, end in steps:
        for r, toks, _ in entries:
            held[r] = held.get(r, 0) + len(toks)
        peak = max(peak, sum((n + round_to - 1) // round_to * round_to for n in held.values()))
        for r in end:
            held.pop(r, None)
    return peak


def collect(replayer, steps: List[Step]) -> Dict[Tuple[str, int], np.ndarray]:
    """Runs the steps through the engine's step function; returns logits by (request, position)."""
    from liyab_b200.engine import StepEntry
    cache = replayer.cache
    out: Dict[Tuple[str, int], np.ndarray] = {}
    held: Dict[str, int] = {}
    for entries, end in steps:
        batch = []
        base = {}
        for r, toks, want in entries:
            if r not in held:
                cache.open(r)
                held[r] = 0
            base[r] = held[r]
            held[r] += len(toks)
            batch.append(StepEntry(request=r, tokens=toks, want=want))
        res = replayer.step(batch)
        if res.logits is not None:
            for (r, idx), row in zip(res.rows, res.logits):
                out[(r, base[r] + idx)] = row.copy()
        for r in end:
            assert cache.length(r) == held.pop(r)
            cache.close(r)
    cache.check()
    return out


def to_jsonl(steps: List[Step]) -> str:
    import json
    lines = []
    for i, (entries, end) in enumerate(steps):
        lines.append(json.dumps({"step": i, "entries": [{"id": r, "tokens": t, "want": w} for r, t, w in entries],
                                 "end": end}))
    return "\n".join(lines) + "\n"


def thin(steps: List[Step], keep) -> List[Step]:
    """The same steps with logits wanted only at the positions `keep(request, position)` says (big vocabularies)."""
    held: Dict[str, int] = {}
    out: List[Step] = []
    for entries, end in steps:
        new = []
        for r, toks, want in entries:
            base = held.get(r, 0)
            new.append((r, toks, [w for w in want if keep(r, base + w)]))
            held[r] = base + len(toks)
        out.append((new, end))
    return out


def kl_and_top1(got: np.ndarray, ref: np.ndarray, margin: float):
    """(KL(plain || engine) of the two softmax distributions, whether the arg-max agrees or None when the plain
    implementation's two best logits lie within `margin`): the reference gates lower precision with the mean of the
    first and the share of the second (tools/liyab_kl.cpp:12-15, 93-99)."""
    ref = ref.astype(np.float64)
    got = got.astype(np.float64)
    lp = ref - ref.max()
    lp -= np.log(np.exp(lp).sum())
    lq = got - got.max()
    lq -= np.log(np.exp(lq).sum())
    kl = float((np.exp(lp) * (lp - lq)).sum())
    top = np.partition(ref, -2)[-2:]
    agree = None if top[1] - top[0] <= margin else bool(np.argmax(got) == np.argmax(ref))
    return kl, agree


def check_rows(got: Dict[Tuple[str, int], np.ndarray], want: Dict[str, np.ndarray], rel_tol: float, max_mean_kl: float = None,
               min_top1: float = None) -> Dict[str, float]:
    """Every row within rel_tol * max|logit| of its sequence; and, where asked, the reference's gate for a lower
    precision: mean KL at most max_mean_kl and the best token the same in at least min_top1 of the rows whose plain
    top-two margin exceeds the tolerance."""
    worst, kls, agrees = 0.0, [], []
    for (r, pos), row in got.items():
        ref = want[r][pos]
        scale = np.abs(want[r]).max()
        err = np.abs(row.astype(np.float64) - ref).max() / scale
        worst = max(worst, err)
        assert err <= rel_tol, f"request {r} position {pos}: relative error {err:.3e} > {rel_tol:.1e}"
        if max_mean_kl is not None:
            kl, agree = kl_and_top1(row, ref, 2 * rel_tol * scale)
            kls.append(kl)
            if agree is not None:
                agrees.append(agree)
    out = {"worst": worst}
    if max_mean_kl is not None:
        out["mean_kl"] = float(np.mean(kls))
        out["top1"] = float(np.mean(agrees)) if agrees else 1.0
        assert out["mean_kl"] <= max_mean_kl, f"mean KL {out['mean_kl']:.3e} > {max_mean_kl:.1e}"
        assert out["top1"] >= min_top1, f"top-1 agreement {out['top1']:.4f} < {min_top1}"
    return out
