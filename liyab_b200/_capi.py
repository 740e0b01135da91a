"""The library's C interface (include/liyab_b200.h) as seen from Python.

Everything the package does goes through these symbols: the engine, and for tools
and tests the engine's layers one by one.  A non-zero status becomes a
`LiyabError` with the library's message; functions that return text are called
with a buffer and, when the text did not fit, once more with a larger one.
"""
from __future__ import annotations

import ctypes as C
import json
from typing import Any

from .csrc.build import load_library
from .status import ErrorCode, LiyabError

i32, i64, u64, f32, f64, vp, cp, sz = C.c_int32, C.c_int64, C.c_uint64, C.c_float, C.c_double, C.c_void_p, C.c_char_p, C.c_size_t
P = C.POINTER


class EngineConfigC(C.Structure):
    _fields_ = [("model_path", cp), ("dtype", cp), ("device", i32), ("context_length", i32), ("max_batched_tokens", i32),
                ("max_sequences", i32), ("page_size", i32), ("num_pages", i32), ("kv_memory_fraction", f32),
                ("cuda_graphs", i32), ("fused_decode", i32), ("pipeline", i32), ("profile_phases", i32)]


class SamplingParamsC(C.Structure):
    _fields_ = [("temperature", f32), ("top_k", i32), ("top_p", f32), ("seed", u64), ("max_tokens", i32), ("ignore_eos", i32)]


class GenerationStatsC(C.Structure):
    _fields_ = [("prompt_tokens", i32), ("generated_tokens", i32), ("prefill_ms", f64), ("decode_ms", f64),
                ("tokens_per_second", f64), ("cancelled", i32), ("kv_cache_bytes", u64), ("ttft_ms", f64), ("preemptions", i32),
                ("finish_reason", i32), ("decode_steps", i32), ("embed_ms", f64), ("norm_ms", f64), ("attention_ms", f64),
                ("dense_ffn_ms", f64), ("lm_head_ms", f64)]


TokenCallback = C.CFUNCTYPE(i32, i32, vp)
LogCallback = C.CFUNCTYPE(None, i32, cp, vp)
TapCallback = C.CFUNCTYPE(None, cp, P(f32), i32, i32, vp)


class RequestC(C.Structure):
    _fields_ = [("tokens", P(i32)), ("n_tokens", sz), ("params", SamplingParamsC), ("callback", TokenCallback), ("user_data", vp),
                ("out_tokens", P(i32)), ("out_capacity", sz), ("n_out", sz), ("status", i32), ("error", C.c_char * 256),
                ("stats", GenerationStatsC)]


class SchedulerStatsC(C.Structure):
    _fields_ = [("steps", u64), ("batched_tokens", u64), ("prefill_tokens", u64), ("decode_tokens", u64), ("preemptions", u64),
                ("finished", u64), ("peak_running", i32), ("histogram", u64 * 7), ("graph_steps", u64), ("fused_steps", u64),
                ("eager_steps", u64), ("graphs_captured", u64), ("kernel_launches", u64), ("pages_in_use", i32),
                ("pages_total", i32), ("h2d_bytes", u64), ("d2h_bytes", u64), ("device_faults", i32)]


class ReplayerOptionsC(C.Structure):
    _fields_ = [("device", i32), ("page_size", i32), ("max_requests", i32), ("num_pages", i32), ("cuda_graphs", i32),
                ("fused_decode", i32), ("max_step_tokens", i32)]


class BenchResultC(C.Structure):
    _fields_ = [("ms_total", f64), ("ms_per_step", f64), ("wall_ms_per_step", f64), ("mean_context", f64), ("kernel_launches", u64),
                ("graph_steps", u64), ("fused_steps", u64), ("eager_steps", u64), ("h2d_bytes_per_step", u64),
                ("d2h_bytes_per_step", u64), ("checksum", u64)]


_TEXT = [cp, sz, P(sz)]        # buffer, size, needed
_SIGNATURES = {
    "lb_version": ([], cp), "lb_set_log_level": ([i32], None), "lb_set_log_callback": ([LogCallback, vp], None),
    "lb_engine_config_default": ([P(EngineConfigC)], None), "lb_sampling_params_default": ([P(SamplingParamsC)], None),
    "lb_engine_create": ([P(EngineConfigC), P(vp)], i32), "lb_engine_destroy": ([vp], None),
    "lb_engine_generate_batch": ([vp, P(RequestC), sz], i32), "lb_engine_cancel": ([vp], None),
    "lb_engine_generate_tokens": ([vp, P(i32), sz, P(SamplingParamsC), TokenCallback, vp, P(i32), sz, P(sz), P(GenerationStatsC)], i32),
    "lb_engine_describe": ([vp, cp, sz], sz), "lb_engine_scheduler_stats": ([vp, P(SchedulerStatsC)], i32),
    "lb_engine_context_length": ([vp], i32), "lb_engine_vocab_size": ([vp], i32), "lb_engine_load_ms": ([vp], f64),
    "lb_engine_weight_bytes": ([vp], u64),
    "lb_load_plugin": ([cp], i32), "lb_supported_architectures": (_TEXT, i32), "lb_config_describe": ([cp] + _TEXT, i32),
    "lb_config_describe_folder": ([cp] + _TEXT, i32), "lb_write_random_model": ([cp, u64, cp, cp], i32),
    "lb_normal_values": ([u64, cp, i64, i64, f64, f64, P(f64)], i32), "lb_uniform_draw": ([u64, u64, u64], f64),
    "lb_safetensors_describe": ([cp] + _TEXT, i32), "lb_safetensors_read": ([cp, cp, vp, sz], i32),
    "lb_safetensors_write": ([cp, sz, P(cp), P(cp), P(i32), P(i64), P(vp), cp], i32),
    "lb_weights_load": ([cp, cp, P(vp)], i32), "lb_weights_free": ([vp], None), "lb_weights_describe": ([vp] + _TEXT, i32),
    "lb_weights_data": ([vp, cp, P(vp), P(sz)], i32),
    "lb_cache_create": ([cp, i32, i32, i32, P(vp)], i32), "lb_cache_destroy": ([vp], None), "lb_cache_describe": ([vp] + _TEXT, i32),
    "lb_cache_open": ([vp, i64], i32), "lb_cache_close": ([vp, i64], i32), "lb_cache_is_open": ([vp, i64], i32),
    "lb_cache_length": ([vp, i64], i64), "lb_cache_reserve": ([vp, i64, i64], i32), "lb_cache_commit": ([vp, i64, i64], i32),
    "lb_cache_truncate": ([vp, i64, i64], i32), "lb_cache_can_reserve": ([vp, sz, P(i64), P(i64), P(i32)], i32),
    "lb_cache_state_slot": ([vp, i64, P(i32)], i32), "lb_cache_block_table": ([vp, i32, sz, P(i64), P(i32), P(i32), sz], i32),
    "lb_cache_slot_mapping": ([vp, i32, i64, i64, i64, P(i32)], i32), "lb_cache_pages": ([vp, P(i32), P(i32), sz], i32),
    "lb_cache_state_slots_free": ([vp], i32), "lb_cache_check": ([vp], i32),
    "lb_scheduler_create": ([vp, i64, i32, i32, i64, P(vp)], i32), "lb_scheduler_destroy": ([vp], None),
    "lb_scheduler_add": ([vp, i64, P(i32), sz, P(SamplingParamsC), TokenCallback, vp], i32), "lb_scheduler_cancel": ([vp, i64], i32),
    "lb_scheduler_has_work": ([vp], i32), "lb_scheduler_plan": ([vp] + _TEXT, i32), "lb_scheduler_begin_step": ([vp, i64], i32),
    "lb_scheduler_finish_step": ([vp, i64, P(i32), sz] + _TEXT, i32), "lb_scheduler_request": ([vp, i64] + _TEXT, i32),
    "lb_scheduler_stats_get": ([vp, P(SchedulerStatsC)], i32),
    "lb_replayer_options_default": ([P(ReplayerOptionsC)], None), "lb_replayer_create": ([cp, cp, i64, P(ReplayerOptionsC), P(vp)], i32),
    "lb_replayer_destroy": ([vp], None), "lb_replayer_cache": ([vp], vp), "lb_replayer_describe": ([vp] + _TEXT, i32),
    "lb_replayer_step": ([vp, sz, P(i64), P(i32), P(i32), P(i32), P(i32), P(f32), sz, P(i32)], i32),
    "lb_replayer_set": ([vp, cp, i32], i32), "lb_replayer_counters": ([vp] + _TEXT, i32),
    "lb_replayer_set_tap": ([vp, TapCallback, vp], i32), "lb_replayer_timer_start": ([vp], i32),
    "lb_replayer_timer_stop": ([vp, P(f64)], i32), "lb_device_status": ([P(i32)], i32), "lb_debug_set_device_status": ([i32, i32], i32),
    "lb_debug_withhold_next": ([i32, i32], i32),
    "lb_replayer_fused_stamps": ([vp, P(C.c_uint64), i32, P(i32)], i32),
    "lb_replayer_bench_decode": ([vp, i32, i32, i32, i32, u64, P(BenchResultC)], i32),
    "lb_replayer_bench_prefill": ([vp, i32, i32, i32, u64, P(BenchResultC)], i32),
}

_lib = None


def lib():
    """The library with argument types declared (built at first use)."""
    global _lib
    if _lib is None:
        l = load_library()
        l.lb_last_error.restype = cp
        for name, (args, res) in _SIGNATURES.items():
            fn = getattr(l, name)
            fn.argtypes = args
            fn.restype = res
        _lib = l
    return _lib


def last_error() -> str:
    return lib().lb_last_error().decode("utf-8", "replace")


def error_from(status: int) -> LiyabError:
    try:
        code = ErrorCode(status)
    except ValueError:
        code = ErrorCode.INTERNAL
    from .status import OutOfPages
    cls = OutOfPages if code == ErrorCode.OUT_OF_MEMORY else LiyabError
    return cls(code, last_error())


def check(status: int) -> None:
    if status != 0:
        raise error_from(status)


def text(fn, *args) -> str:
    """Calls a function of the (..., buffer, size, needed) shape and returns its text."""
    size = 1 << 16
    while True:
        buf = C.create_string_buffer(size)
        needed = sz(0)
        check(fn(*args, buf, size, C.byref(needed)))
        if needed.value < size:
            return buf.value.decode("utf-8")
        size = needed.value + 1


def json_of(fn, *args) -> Any:
    return json.loads(text(fn, *args))


def b(s: str) -> bytes:
    return s.encode("utf-8")
