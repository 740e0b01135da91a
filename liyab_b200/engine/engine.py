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
from .step import StepEntry, Stepper


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
        """Steps until the scheduler has no work (or all of `watch` have finished)."""
        sched = self.scheduler
        t_start = time.perf_counter()
        times: Dict[Hashable, Dict[str, float]] = {}
        self._times = times
        idle = 0
        while sched.has_work():
            if watch is not None and all(r.state == RequestState.FINISHED for r in watch):
                break
            plan, _ = sched.plan()
            if not plan.entries:
                idle += 1
                if idle > 2 and sched.has_work():
                    raise LiyabError(ErrorCode.INTERNAL, "the scheduler has work but plans no step")
                continue
            idle = 0
            t0 = time.perf_counter()
            entries = [StepEntry(request=e.request.id, tokens=e.tokens, want=[e.count - 1] if e.sample else [])
                       for e in plan.entries]
            sampling = [e.request for e in plan.entries if e.sample]
            out = self.stepper.step(entries)
            ids: List[int] = []
            if sampling:
                self.sampler.sample(out.logits, [r.params for r in sampling], [r.next_uniform() for r in sampling])
                ids = self.sampler.to_host(len(sampling))
            else:
                torch.cuda.current_stream().synchronize()
            dt = (time.perf_counter() - t0) * 1e3
            for e in plan.entries:
                t = times.setdefault(e.request.id, dict(prefill=0.0, decode=0.0, ttft=0.0))
                first = len(e.request.tokens) == len(e.request.prompt)
                if e.start + e.count <= len(e.request.prompt) or first:
                    t["prefill"] += dt
                    if e.sample and first:
                        t["ttft"] = (time.perf_counter() - t_start) * 1e3
                else:
                    t["decode"] += dt
            sched.update(plan, ids)

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
