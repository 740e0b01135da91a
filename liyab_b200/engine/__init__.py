"""The engine, the scheduler and the step function as seen from Python.

`Engine` mirrors the reference's public surface where it has one
(`Engine::create(config)`, `generate_tokens(tokens, params, callback)`, `cancel`,
`describe`, generation statistics: include/liyab/engine.h:634-1052,
include/liyab/liyab_c_api.h:137-189, 223-275) through the library's C interface.
`Replayer` is a model with a cache and the step function (what bin/trace_run and the
tests drive); `Scheduler` is the scheduler over a cache manager, for tests that play
the step function themselves.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np

from .. import _capi
from ..cache import CacheManager
from ..sampling import SamplingParams
from ..status import ErrorCode, LiyabError, invalid_argument

FINISH_REASONS = ["unfinished", "eos", "length", "context", "stopped", "cancelled", "error"]


@dataclass
class EngineConfig:
    """Options of `Engine`; names follow the reference's engine config and CLI where they exist
    (`context_length` is --ctx, tools/liyab_cli.cpp:242-334)."""
    model: str = ""                    # folder with config.json and model.safetensors
    dtype: str = "bfloat16"            # bfloat16 | float32
    device: int = 0
    context_length: int = 0            # 0: the model's positions
    max_batched_tokens: int = 2048     # token budget of one step
    max_requests: int = 64             # requests served together
    page_size: int = 16                # positions per cache page
    num_pages: int = 0                 # 0: enough for max_requests full contexts, within kv_memory_fraction
    kv_memory_fraction: float = 0.5    # of the free device memory, at most, for the cache when num_pages is 0
    cuda_graphs: bool = True           # replay captured graphs for steps whose shape repeats
    fused_decode: bool = False         # decode steps of up to 16 requests as one persistent kernel (bfloat16); off: the part-by-part path is faster
    pipeline: bool = True              # plan and launch step n+1 while step n runs (tokens stay on the device)
    profile_phases: bool = False       # time every step's phases (slower)


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
    decode_steps: int = 0
    phase_ms: Dict[str, float] = field(default_factory=dict)


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str
    stats: GenerationStats = field(default_factory=GenerationStats)
    error: Optional[LiyabError] = None


def _stats(s: "_capi.GenerationStatsC") -> GenerationStats:
    return GenerationStats(
        prompt_tokens=s.prompt_tokens, generated_tokens=s.generated_tokens, prefill_ms=s.prefill_ms, decode_ms=s.decode_ms,
        ttft_ms=s.ttft_ms, tokens_per_second=s.tokens_per_second, kv_cache_bytes=s.kv_cache_bytes, cancelled=bool(s.cancelled),
        preemptions=s.preemptions, decode_steps=s.decode_steps,
        phase_ms={"embed": s.embed_ms, "norm": s.norm_ms, "attention": s.attention_ms, "dense_ffn": s.dense_ffn_ms, "lm_head": s.lm_head_ms})


def _scheduler_stats(s: "_capi.SchedulerStatsC") -> Dict[str, Any]:
    d = {name: getattr(s, name) for name, _ in s._fields_ if name != "histogram"}
    d["histogram"] = list(s.histogram)
    return d


class Engine:
    def __init__(self, config: Optional[EngineConfig] = None, **overrides):
        cfg = config or EngineConfig()
        for k, v in overrides.items():
            if not hasattr(cfg, k):
                raise invalid_argument(f"unknown engine option {k!r}")
            setattr(cfg, k, v)
        self.config = cfg
        self._lib = _capi.lib()
        c = _capi.EngineConfigC()
        self._lib.lb_engine_config_default(C.byref(c))
        self._keep = (_capi.b(cfg.model), _capi.b(cfg.dtype))
        c.model_path, c.dtype = self._keep
        c.device, c.context_length, c.max_batched_tokens = cfg.device, cfg.context_length, cfg.max_batched_tokens
        c.max_sequences, c.page_size, c.num_pages = cfg.max_requests, cfg.page_size, cfg.num_pages
        c.kv_memory_fraction = cfg.kv_memory_fraction
        c.cuda_graphs, c.fused_decode, c.pipeline = int(cfg.cuda_graphs), int(cfg.fused_decode), int(cfg.pipeline)
        c.profile_phases = int(cfg.profile_phases)
        h = C.c_void_p()
        _capi.check(self._lib.lb_engine_create(C.byref(c), C.byref(h)))
        self._h = h
        self.max_positions = self._lib.lb_engine_context_length(h)
        self.vocab_size = self._lib.lb_engine_vocab_size(h)
        self.load_ms = self._lib.lb_engine_load_ms(h)

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.lb_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def describe(self) -> str:
        buf = C.create_string_buffer(2048)
        self._lib.lb_engine_describe(self._h, buf, 2048)
        return buf.value.decode()

    def weight_bytes(self) -> int:
        return int(self._lib.lb_engine_weight_bytes(self._h))

    def stats(self) -> Dict[str, Any]:
        """Scheduler and step counters since the engine was created (steps, batched tokens and their histogram,
        preemptions, graph / fused / part-by-part steps, kernel launches, pages in use)."""
        s = _capi.SchedulerStatsC()
        _capi.check(self._lib.lb_engine_scheduler_stats(self._h, C.byref(s)))
        return _scheduler_stats(s)

    def cancel(self) -> None:
        self._lib.lb_engine_cancel(self._h)

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
        reqs = (_capi.RequestC * max(1, n))()
        keep = []
        for i, (p, sp, cb) in enumerate(zip(prompts, params, callbacks)):
            ids = np.ascontiguousarray(p, dtype=np.int32)
            out = np.zeros(max(1, sp.max_tokens), dtype=np.int32)
            keep += [ids, out]
            q = reqs[i]
            q.tokens, q.n_tokens = ids.ctypes.data_as(C.POINTER(C.c_int32)), len(ids)
            q.params = sp.to_c()
            if cb is not None:
                fn = _capi.TokenCallback(lambda token, _user, cb=cb: 0 if cb(int(token)) is False else 1)
                keep.append(fn)
                q.callback = fn
            q.out_tokens, q.out_capacity = out.ctypes.data_as(C.POINTER(C.c_int32)), len(out)
        _capi.check(self._lib.lb_engine_generate_batch(self._h, reqs, n))
        results = []
        for i in range(n):
            q = reqs[i]
            out = keep[2 * i + 1] if callbacks[i] is None else None
            toks = np.ctypeslib.as_array(q.out_tokens, shape=(q.out_capacity,))[:q.n_out].tolist()
            err = LiyabError(ErrorCode(q.status), q.error.decode("utf-8", "replace")) if q.status != 0 else None
            results.append(GenerationResult(tokens=toks, finish_reason=FINISH_REASONS[q.stats.finish_reason], stats=_stats(q.stats), error=err))
        return results


def generate(model: str, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None, **options) -> List[List[int]]:
    """One call: load `model` (a folder), generate for every prompt, return the new token ids."""
    engine = Engine(EngineConfig(model=model, **options))
    try:
        return [r.tokens for r in engine.generate_batch(prompts, params)]
    finally:
        engine.close()


# ---- the step function ---------------------------------------------------------------------------------

@dataclass
class StepEntry:
    """A request's next tokens and the places among them whose logits are wanted."""
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class StepOutput:
    logits: Optional[np.ndarray]                                       # [R, vocab] float32
    rows: List[Tuple[Hashable, int]] = field(default_factory=list)     # (request, index among its tokens) per row


class Replayer:
    """A model on the device, a cache sized for `max_tokens` live tokens and the step function."""

    def __init__(self, model_dir: str, dtype: str, max_tokens: int, page_size: int = 16, max_requests: int = 16, num_pages: int = 0,
                 cuda_graphs: bool = False, fused_decode: bool = False, max_step_tokens: int = 0, device: int = 0):
        self._lib = _capi.lib()
        o = _capi.ReplayerOptionsC(device, page_size, max_requests, num_pages, int(cuda_graphs), int(fused_decode), max_step_tokens)
        h = C.c_void_p()
        _capi.check(self._lib.lb_replayer_create(_capi.b(model_dir), _capi.b(dtype), max_tokens, C.byref(o), C.byref(h)))
        self._h = h
        self.cache = CacheManager(_borrowed=C.c_void_p(self._lib.lb_replayer_cache(h)))
        self.info = self.describe()
        self.vocab_size = self.info["vocab_size"]
        self._tap = None

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.lb_replayer_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def describe(self) -> Dict[str, Any]:
        return _capi.json_of(self._lib.lb_replayer_describe, self._h)

    def counters(self) -> Dict[str, int]:
        return _capi.json_of(self._lib.lb_replayer_counters, self._h)

    def set(self, option: str, value: int) -> None:
        _capi.check(self._lib.lb_replayer_set(self._h, _capi.b(option), int(value)))

    def fused_stamps(self) -> np.ndarray:
        """The last one-kernel decode step's time stamps in ns (after `set("fused_stamps", 1)`): entry b = block 0 left
        grid barrier b; 128 + 8 * layer + mark = marks inside the phases; 256 + 160 * j + block = every block's
        arrival at barrier j of layer 5.  Entries never written are 0."""
        n = C.c_int32(0)
        _capi.check(self._lib.lb_replayer_fused_stamps(self._h, None, 0, C.byref(n)))
        out = np.zeros(n.value, dtype=np.uint64)
        if n.value:
            _capi.check(self._lib.lb_replayer_fused_stamps(self._h, out.ctypes.data_as(C.POINTER(C.c_uint64)), n.value, C.byref(n)))
        return out

    def set_tap(self, fn: Optional[Callable[[str, np.ndarray], None]]) -> None:
        """`fn(name, rows)` is called with every part's output (float32 on the host) of the following steps."""
        if fn is None:
            self._tap = None
            _capi.check(self._lib.lb_replayer_set_tap(self._h, _capi.TapCallback(), None))
            return
        def tap(name, data, n_rows, n_cols, _user):
            fn(name.decode(), np.ctypeslib.as_array(data, shape=(n_rows, n_cols)).copy())
        self._tap = _capi.TapCallback(tap)
        _capi.check(self._lib.lb_replayer_set_tap(self._h, self._tap, None))

    def step(self, entries: Sequence[StepEntry], fetch: bool = True) -> StepOutput:
        n = len(entries)
        ids = (C.c_int64 * max(1, n))(*[self.cache.ids(e.request) for e in entries])
        n_tok = (C.c_int32 * max(1, n))(*[len(e.tokens) for e in entries])
        n_want = (C.c_int32 * max(1, n))(*[len(e.want) for e in entries])
        toks = np.ascontiguousarray([t for e in entries for t in e.tokens], dtype=np.int32)
        want = np.ascontiguousarray([w for e in entries for w in e.want], dtype=np.int32)
        rows = [(e.request, int(w)) for e in entries for w in e.want]
        logits = np.empty((len(rows), self.vocab_size), dtype=np.float32) if fetch and rows else None
        n_rows = C.c_int32(0)
        p32 = C.POINTER(C.c_int32)
        _capi.check(self._lib.lb_replayer_step(
            self._h, n, ids, n_tok, toks.ctypes.data_as(p32), n_want, want.ctypes.data_as(p32),
            logits.ctypes.data_as(C.POINTER(C.c_float)) if logits is not None else None, logits.size if logits is not None else 0,
            C.byref(n_rows)))
        return StepOutput(logits=logits, rows=rows)

    def bench_decode(self, batch: int, prompt_len: int, steps: int, warmup: int, seed: int = 0) -> Dict[str, Any]:
        r = _capi.BenchResultC()
        _capi.check(self._lib.lb_replayer_bench_decode(self._h, batch, prompt_len, steps, warmup, seed, C.byref(r)))
        return {name: getattr(r, name) for name, _ in r._fields_}

    def bench_prefill(self, n_seq: int, seq_len: int, repeats: int = 5, seed: int = 1) -> Dict[str, Any]:
        r = _capi.BenchResultC()
        _capi.check(self._lib.lb_replayer_bench_prefill(self._h, n_seq, seq_len, repeats, seed, C.byref(r)))
        return {name: getattr(r, name) for name, _ in r._fields_}


def device_status() -> Tuple[int, int]:
    """(tcgen05/TMA waits, fused step's barrier): 0 unless a bounded wait inside a kernel ran out since the last
    call.  Synchronises the device."""
    words = (C.c_int32 * 2)()
    _capi.check(_capi.lib().lb_device_status(words))
    return words[0], words[1]


def withhold_next(which: int, on: bool = True) -> None:
    """The next launch of kernel family `which` (0: the one-tile tcgen05 product, 1: the one-kernel decode step) meets
    a wait that nothing ends, once: its bounded wait runs to its limit (about two seconds), sets the status word and
    the kernel returns.  `on=False` takes back an order that no launch has used.  For tests of that path; the device
    stays usable."""
    _capi.check(_capi.lib().lb_debug_withhold_next(which, 1 if on else 0))


def set_device_status(which: int, value: int) -> None:
    """Writes a device status word as a kernel whose bounded wait ran out would (tests of the engine's handling)."""
    _capi.check(_capi.lib().lb_debug_set_device_status(which, value))


def set_log(level: int, callback: Optional[Callable[[int, str], None]] = None) -> None:
    """Diagnostics: level 0 debug, 1 info, 2 warn (default), 3 error, 4 off; `callback(level, message)` receives the
    messages at or above it instead of stderr (None: stderr again)."""
    l = _capi.lib()
    l.lb_set_log_level(level)
    global _log_keep
    if callback is None:
        _log_keep = None
        l.lb_set_log_callback(_capi.LogCallback(), None)
    else:
        _log_keep = _capi.LogCallback(lambda lvl, msg, _user: callback(int(lvl), msg.decode("utf-8", "replace")))
        l.lb_set_log_callback(_log_keep, None)


_log_keep = None


# ---- the scheduler, for tests that play the step function ---------------------------------------------------

@dataclass
class Request:
    id: Hashable
    prompt: List[int]
    params: SamplingParams
    callback: Optional[Callable[[int], bool]] = None
    _sched: Any = None

    def _info(self) -> Dict[str, Any]:
        return self._sched._request_info(self.id)

    @property
    def tokens(self) -> List[int]:
        return self._info()["tokens"] if self._sched else list(self.prompt)

    @property
    def generated(self) -> List[int]:
        return self.tokens[len(self.prompt):]

    @property
    def state(self) -> str:
        return self._info()["state"] if self._sched else "waiting"

    @property
    def finish_reason(self) -> Optional[str]:
        return self._info()["finish_reason"] if self._sched else None

    @property
    def n_computed(self) -> int:
        return self._info()["n_computed"]

    @property
    def preemptions(self) -> int:
        return self._info()["preemptions"]

    @property
    def error(self) -> Optional[LiyabError]:
        i = self._info()
        return LiyabError(ErrorCode(i["error_code"]), i["error"]) if i["error_code"] else None

    @property
    def seed(self) -> int:
        return self._info()["seed"]

    @property
    def stream(self) -> int:
        return self._info()["stream"]


@dataclass
class PlannedEntry:
    request: Request
    start: int
    count: int
    sample: bool
    tokens: List[int]


@dataclass
class StepPlan:
    entries: List[PlannedEntry]
    preempted: List[Request] = field(default_factory=list)
    id: int = -1


class Scheduler:
    def __init__(self, cache: CacheManager, max_positions: int, max_batched_tokens: int = 2048, max_requests: int = 64,
                 eos_token_id: Optional[int] = None):
        self._lib = _capi.lib()
        self.cache = cache
        h = C.c_void_p()
        _capi.check(self._lib.lb_scheduler_create(cache._h, max_positions, max_batched_tokens, max_requests,
                                                  -1 if eos_token_id is None else eos_token_id, C.byref(h)))
        self._h = h
        self._requests: Dict[Hashable, Request] = {}
        self._by_id: Dict[int, Request] = {}
        self._keep: List[Any] = []

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.lb_scheduler_destroy(self._h)
            self._h = None

    def _request_info(self, rid: Hashable) -> Dict[str, Any]:
        return _capi.json_of(self._lib.lb_scheduler_request, self._h, self.cache.ids(rid))

    def add(self, request: Request) -> None:
        ids = np.ascontiguousarray(request.prompt, dtype=np.int32)
        cb = _capi.TokenCallback()
        if request.callback is not None:
            cb = _capi.TokenCallback(lambda token, _user, f=request.callback: 0 if f(int(token)) is False else 1)
            self._keep.append(cb)
        p = request.params.to_c()
        _capi.check(self._lib.lb_scheduler_add(self._h, self.cache.ids(request.id), ids.ctypes.data_as(C.POINTER(C.c_int32)), len(ids),
                                               C.byref(p), cb, None))
        request._sched = self
        self._requests[request.id] = request
        self._by_id[self.cache.ids(request.id)] = request

    def has_work(self) -> bool:
        return bool(self._lib.lb_scheduler_has_work(self._h))

    def cancel(self, request_id: Hashable) -> None:
        _capi.check(self._lib.lb_scheduler_cancel(self._h, self.cache.ids(request_id)))

    def plan(self) -> Tuple[StepPlan, List[Request]]:
        raw = _capi.json_of(self._lib.lb_scheduler_plan, self._h)
        entries = [PlannedEntry(self._by_id[e["request"]], e["start"], e["count"], e["sample"], e["tokens"]) for e in raw["entries"]]
        return (StepPlan(entries, [self._by_id[i] for i in raw["preempted"]], raw["plan"]), [self._by_id[i] for i in raw["finished"]])

    def begin_step(self, plan: StepPlan) -> None:
        _capi.check(self._lib.lb_scheduler_begin_step(self._h, plan.id))

    def finish_step(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        ids = np.ascontiguousarray(sampled, dtype=np.int32)
        done = _capi.json_of(self._lib.lb_scheduler_finish_step, self._h, plan.id, ids.ctypes.data_as(C.POINTER(C.c_int32)), len(ids))
        return [self._by_id[i] for i in done]

    def update(self, plan: StepPlan, sampled: Sequence[int]) -> List[Request]:
        self.begin_step(plan)
        return self.finish_step(plan, sampled)

    @property
    def stats(self) -> Dict[str, Any]:
        s = _capi.SchedulerStatsC()
        _capi.check(self._lib.lb_scheduler_stats_get(self._h, C.byref(s)))
        return _scheduler_stats(s)


__all__ = ["Engine", "EngineConfig", "GenerationResult", "GenerationStats", "generate", "StepEntry", "StepOutput", "Replayer",
           "device_status", "set_device_status", "withhold_next", "set_log", "Request", "PlannedEntry", "StepPlan", "Scheduler", "FINISH_REASONS"]
