"""The Python entry point: load a model folder, generate tokens.

`Engine` mirrors the reference's public surface where it has one:
`Engine::create(config)`, `generate_tokens(tokens, params, callback)`, `cancel`,
`describe`, generation statistics (include/liyab/engine.h:634-1052,
include/liyab/liyab_c_api.h:137-189, 223-275).  Token ids go in and come out;
there is no tokenizer.  Several requests are served together by the scheduler
(`generate_batch`), each with its own sampling options.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Hashable, List, Optional, Sequence

import torch

from ..cache.pages import CacheManager
from ..models.loading import load_model
from ..sampling.params import SamplingParams
from ..sampling.sampler import DeviceSampler
from ..status import ErrorCode, LiyabError, invalid_argument
from .scheduler import Request, RequestState, Scheduler
from .step import DeviceTokens, StepEntry, Stepper


@dataclass
class EngineConfig:
    """Options of `Engine`; names follow the reference's engine config and CLI where they exist
    (`context_length` is --ctx, tools/liyab_cli.cpp:242-334)."""
    model: str = ""                    # folder with config.json and model.safetensors
    dtype: str = "bfloat16"            # bfloat16 | float32
    device: str = "cuda:0"
    context_length: int = 0            # 0: the model's positions
    max_batched_tokens: int = 2048     # token budget of one step
    max_requests: int = 64             # requests served together
    page_size: int = 16                # positions per cache page
    num_pages: int = 0                 # 0: enough for max_requests full contexts, within kv_memory_fraction
    kv_memory_fraction: float = 0.5    # of the free device memory, at most, for the cache when num_pages is 0
    cuda_graphs: bool = True           # replay captured graphs for decode-only steps
    fused_decode: bool = True          # one persistent kernel for decode steps of up to 16 requests (bfloat16)
    pipeline: bool = True              # plan and launch step n+1 while step n runs (tokens stay on the device)


@dataclass
class GenerationStats:
    """Per request, in the reference's names (include/liyab/liyab_c_api.h:137-189)."""
    prompt_tokens: int = 0
    generated_tokens: int = 0
    prefill_ms: float = 0.0
    decode_ms: float = 0.0
    ttft_ms: float = 0.0
    tokens_per_second: float = 0.0
    kv_cache_bytes: int = 0
    cancelled: bool = False
    preemptions: int = 0


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str
    stats: GenerationStats = field(default_factory=GenerationStats)
    error: Optional[LiyabError] = None


class Engine:
    def __init__(self, config: Optional[EngineConfig] = None, **overrides):
        cfg = config or EngineConfig()
        for k, v in overrides.items():
            if not hasattr(cfg, k):
                raise invalid_argument(f"unknown engine option {k!r}")
            setattr(cfg, k, v)
        if not cfg.model:
            raise invalid_argument("EngineConfig.model (a model folder) is required")
        self.config = cfg
        t0 = time.perf_counter()
        self.model, self.model_config = load_model(cfg.model, cfg.dtype, cfg.device)
        self.device = self.model.runtime.device
        self.max_positions = self.model.max_positions
        if cfg.context_length:
            self.max_positions = min(self.max_positions, cfg.context_length)
        kv_needs, state_needs = self.model.kv_needs(), self.model.state_needs()
        probe = CacheManager(kv_needs, state_needs, cfg.page_size, 1, 1, dtype=self.model.runtime.dtype, device=None)
        per_page = max(1, probe.bytes_per_token() * cfg.page_size)
        num_pages = cfg.num_pages
        if num_pages <= 0:
            want = cfg.max_requests * ((self.max_positions + cfg.page_size - 1) // cfg.page_size)
            free, _ = torch.cuda.mem_get_info(self.device)
            num_pages = max(1, min(want, int(free * cfg.kv_memory_fraction) // per_page))
        self.cache = CacheManager(kv_needs, state_needs, cfg.page_size, num_pages, cfg.max_requests,
                                  dtype=self.model.runtime.dtype, device=self.device)
        self.stepper = Stepper(self.model, self.cache, max_step_tokens=cfg.max_batched_tokens,
                               cuda_graphs=cfg.cuda_graphs, max_positions=self.max_positions,
                               fused_decode=cfg.fused_decode)
        self.scheduler = Scheduler(self.cache, self.max_positions, cfg.max_batched_tokens, cfg.max_requests,
                                   eos_token_id=self.model.spec.eos_token_id)
        self.sampler = DeviceSampler(self.device, cfg.max_requests)
        self.load_ms = (time.perf_counter() - t0) * 1e3
        self._next_id = 0

    # -- description -------------------------------------------------------------

    def describe(self) -> str:
        """One line about the loaded model (the reference prints the like at load: src/core/transformer.cpp:880-884)."""
        s, c = self.model.spec, self.cache
        return (f"{s.architecture}: {len(s.run_order)} layers, width {s.hidden}, vocab {s.vocab_size}, "
                f"{self.max_positions} positions, {self.config.dtype}, weights {self.model.weight_bytes() / 2**20:.1f} MiB, "
                f"cache {sum(g.pool.num_pages for g in c.groups)} pages x {c.page_size} positions "
                f"({c.bytes_per_token()} B/position), up to {self.config.max_requests} requests, "
                f"{self.config.max_batched_tokens} tokens a step")

    # -- generation -----------------------------------------------------------------

    def generate_tokens(self, tokens: Sequence[int], params: Optional[SamplingParams] = None,
                        callback: Optional[Callable[[int], bool]] = None) -> GenerationResult:
        """Generates after the prompt `tokens`; `callback(token)` may return False to stop."""
        return self.generate_batch([tokens], [params or SamplingParams()], [callback])[0]

    def generate_batch(self, prompts: Sequence[Sequence[int]], params=None, callbacks=None) -> List[GenerationResult]:
        """Serves all prompts together; `params` is one SamplingParams or one per prompt."""
        n = len(prompts)
        if params is None:
            params = SamplingParams()
        if isinstance(params, SamplingParams):
            params = [params] * n
        callbacks = callbacks or [None] * n
        if len(params) != n or len(callbacks) != n:
            raise invalid_argument("params and callbacks must match the prompts in number")
        vocab = self.model.spec.vocab_size
        requests = []
        for p, sp, cb in zip(prompts, params, callbacks):
            p = [int(t) for t in p]
            if any(t < 0 or t >= vocab for t in p):
                raise invalid_argument(f"a prompt has a token id outside [0, {vocab})")
            r = Request(id=f"g{self._next_id}", prompt=p, params=sp, callback=cb)
            self._next_id += 1
            self.scheduler.add(r)
            requests.append(r)
        self.run(requests)
        return [self._result(r) for r in requests]

    def cancel(self, request_id: Hashable) -> None:
        self.scheduler.cancel(request_id)

    def run(self, watch: Optional[Sequence[Request]] = None) -> None:
        """Steps until the scheduler has no work (or all of `watch` have finished).

        With `pipeline` the host runs one step ahead of the GPU: step n+1 is planned, laid out and launched
        while step n computes; the ids step n samples go into step n+1's token array on the device, and
        reach the host (for end-of-sequence checks, callbacks and the results) while step n+1 runs.
        Every step still copies its layout from pinned host memory to the device and its ids back."""
        sched = self.scheduler
        self._times = times = {}
        self._t_start = self._t_last = time.perf_counter()
        inflight = None
        idle = 0
        while True:
            watching = watch is not None and all(r.state == RequestState.FINISHED for r in watch)
            launched, progressed = None, inflight is not None
            if sched.has_work() and not watching:
                plan, _ = sched.plan()
                if plan.entries:
                    launched, progressed = self._launch(plan), True
                    sched.begin_step(plan)
                    if not self.config.pipeline:
                        self._resolve(launched)
                        launched = None
            if inflight is not None:
                self._resolve(inflight)
            inflight = launched
            if inflight is None and (not sched.has_work() or
                                     (watch is not None and all(r.state == RequestState.FINISHED for r in watch))):
                break
            idle = 0 if progressed else idle + 1
            if idle > 3:
                raise LiyabError(ErrorCode.INTERNAL, "the scheduler has work but plans no step")

    def _launch(self, plan):
        """Lays the plan out, launches its kernels and its sampling, and starts the copy of the ids to the host."""
        sampling = [e.request for e in plan.entries if e.sample]
        index, entries, on_device = [], [], False
        for e in plan.entries:
            toks = e.tokens
            if e.count == 1 and toks[0] < 0:           # sampled by the step in flight: still on the device
                index.append(e.request.sample_slot)
                toks = [0]
                on_device = True
            else:
                index.append(-1)
            entries.append(StepEntry(request=e.request.id, tokens=toks, want=[e.count - 1] if e.sample else []))
        uniforms = [r.next_uniform() for r in sampling]
        out = self.stepper.step(entries, DeviceTokens(self.sampler.out_ids, index) if on_device else None)
        ticket = None
        if sampling:
            self.sampler.sample(out.logits, [r.params for r in sampling], uniforms)
            ticket = self.sampler.fetch_async(len(sampling))
            for slot, r in enumerate(sampling):
                r.sample_slot = slot
        return plan, sampling, ticket

    def _resolve(self, launched) -> None:
        """Waits for a launched step's ids and lets the scheduler finish the step."""
        plan, sampling, ticket = launched
        if ticket is not None:
            ids = self.sampler.wait(ticket, len(sampling))
        else:
            ids = []
            torch.cuda.current_stream().synchronize()
        now = time.perf_counter()
        dt, self._t_last = (now - self._t_last) * 1e3, now
        for e in plan.entries:
            t = self._times.setdefault(e.request.id, dict(prefill=0.0, decode=0.0, ttft=0.0))
            first = e.sample and e.token_index == len(e.request.prompt)
            if e.start + e.count <= len(e.request.prompt) or first:
                t["prefill"] += dt
                if first:
                    t["ttft"] = (now - self._t_start) * 1e3
            else:
                t["decode"] += dt
        self.scheduler.finish_step(plan, ids)

    def _result(self, r: Request) -> GenerationResult:
        t = getattr(self, "_times", {}).get(r.id, dict(prefill=0.0, decode=0.0, ttft=0.0))
        gen = r.generated
        stats = GenerationStats(
            prompt_tokens=len(r.prompt), generated_tokens=len(gen), prefill_ms=t["prefill"], decode_ms=t["decode"],
            ttft_ms=t["ttft"], tokens_per_second=(max(0, len(gen) - 1) / (t["decode"] / 1e3)) if t["decode"] > 0 else 0.0,
            kv_cache_bytes=self.cache.bytes_per_token() * (len(r.prompt) + len(gen)),
            cancelled=r.finish_reason == "cancelled", preemptions=r.preemptions)
        return GenerationResult(tokens=list(gen), finish_reason=r.finish_reason or "unfinished", stats=stats, error=r.error)


def generate(model: str, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None, **options
             ) -> List[List[int]]:
    """One call: load `model` (a folder), generate for every prompt, return the new token ids."""
    engine = Engine(EngineConfig(model=model, **options))
    return [r.tokens for r in engine.generate_batch(prompts, params)]
