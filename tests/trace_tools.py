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
