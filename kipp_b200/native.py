"""ctypes declarations of the host core's C interface (csrc/host/kipp_b200.h)
and the mapping of its result codes to Python exceptions.

The engine itself is the C++ library; the Python package is a face of it: it
writes model folders, turns Python objects into the library's structures and
wraps device memory the library owns as torch tensors.
"""
from __future__ import annotations

import ctypes
from ctypes import (POINTER, Structure, c_char_p, c_double, c_float, c_int, c_int32, c_int64, c_longlong, c_size_t,
                    c_uint64, c_void_p)

OK, E_ARGUMENT, E_CONFIG, E_WEIGHTS, E_IO, E_UNSUPPORTED, E_OUT_OF_PAGES, E_OUT_OF_SLOTS = range(8)
E_MEMORY, E_KERNEL, E_CUDA, E_STATE, E_BUILD = range(8, 13)

DTYPE_F32, DTYPE_BF16, DTYPE_F16, DTYPE_I32, DTYPE_I64, DTYPE_I16, DTYPE_I8, DTYPE_U8 = range(8)


class KernelError(RuntimeError):
    """A kernel refused its sizes, reported a refused access, or a wait ran out."""


class EngineOptions(Structure):
    _fields_ = [("dtype", c_int), ("device", c_int), ("page_size", c_int), ("cache_tokens", c_longlong),
                ("max_requests", c_int), ("max_batch_tokens", c_int), ("max_logit_rows", c_int),
                ("cuda_graphs", c_int), ("kv_round_bf16", c_int), ("own_length_splits", c_int)]


class TensorInfo(Structure):
    _fields_ = [("name", c_char_p), ("dtype", c_int), ("ndim", c_int), ("shape", POINTER(c_int64)),
                ("data", c_void_p), ("bytes", c_size_t)]


class TensorView(Structure):
    _fields_ = [("data", c_void_p), ("on_device", c_int), ("dtype", c_int), ("ndim", c_int), ("shape", c_int64 * 8)]


class ExternalCall(Structure):
    _fields_ = [("role", c_int), ("tokens", c_int), ("entries", c_int), ("layer", c_int), ("cache", c_int),
                ("writes_cache", c_int), ("token_ids", c_void_p), ("positions", c_void_p),
                ("entry_of_token", c_void_p), ("q_start", c_void_p), ("context_len", c_void_p), ("slots", c_void_p),
                ("host_q_lens", POINTER(c_int)), ("host_context_len", POINTER(c_int)), ("host_slots", POINTER(c_int)),
                ("input", c_void_p), ("input_dtype", c_int), ("input_cols", c_longlong), ("residual", c_void_p),
                ("hidden", c_longlong), ("output", c_void_p), ("rows", c_void_p), ("n_rows", c_int),
                ("state", c_void_p), ("state_bytes", c_longlong), ("max_requests", c_int), ("stream", c_void_p)]


EXTERNAL_FORWARD = ctypes.CFUNCTYPE(c_int, c_void_p, POINTER(ExternalCall))
TENSOR_PROVIDER = ctypes.CFUNCTYPE(c_int, c_void_p, c_char_p, POINTER(TensorView))


class ExternalPart(Structure):
    _fields_ = [("user", c_void_p), ("forward", EXTERNAL_FORWARD)]


class StepEntryC(Structure):
    _fields_ = [("request", c_int64), ("tokens", POINTER(c_int32)), ("n_tokens", c_int),
                ("want", POINTER(c_int32)), ("n_want", c_int)]


class SampleParams(Structure):
    _fields_ = [("temperature", c_float), ("top_p", c_float), ("top_k", c_int), ("min_p", c_float),
                ("frequency_penalty", c_float), ("presence_penalty", c_float), ("repetition_penalty", c_float),
                ("recent_tokens", POINTER(c_int32)), ("recent_count", c_int),
                ("logit_bias_tokens", POINTER(c_int32)), ("logit_bias_values", POINTER(c_float)),
                ("logit_bias_count", c_int)]


class SchedulerOptions(Structure):
    _fields_ = [("max_batch_tokens", c_int), ("chunk", c_int), ("max_running", c_int), ("max_positions", c_int),
                ("preempt", c_int)]


class GenerationRequest(Structure):
    _fields_ = [("id", c_int64), ("prompt", POINTER(c_int32)), ("n_prompt", c_int), ("max_new_tokens", c_int),
                ("sampling", SampleParams), ("seed", c_uint64), ("stop_tokens", POINTER(c_int32)),
                ("n_stop_tokens", c_int)]


class GenerationState(Structure):
    _fields_ = [("id", c_int64), ("finished", c_int), ("reason", c_int), ("n_tokens", c_int), ("preemptions", c_int)]


class PlanEntry(Structure):
    _fields_ = [("id", c_int64), ("first", c_int), ("n_tokens", c_int), ("want_last", c_int)]


_vp, _i, _ll = c_void_p, c_int, c_longlong
_ip, _llp = POINTER(c_int), POINTER(c_longlong)
_cpp = POINTER(c_char_p)

_SIGNATURES = {
    "kipp_result_name": (c_char_p, [_i]),
    "kipp_last_error": (c_char_p, []),
    "kipp_engine_default_options": (None, [POINTER(EngineOptions)]),
    "kipp_plan_from_config": (_i, [c_char_p, _cpp]),
    "kipp_config_normalize": (_i, [c_char_p, _cpp]),
    "kipp_plan_tensor_specs": (_i, [c_char_p, _cpp]),
    "kipp_part_tensor_specs": (_i, [c_char_p, c_char_p, _cpp]),
    "kipp_attention_split_length": (_i, [_i, _i, _i, _i, _i]),
    "kipp_attention_stream_pays": (_i, [_i, ctypes.POINTER(ctypes.c_int), _i, _i]),
    "kipp_registered": (c_char_p, []),
    "kipp_weights_open": (_i, [c_char_p, POINTER(_vp)]),
    "kipp_weights_close": (None, [_vp]),
    "kipp_weights_count": (_i, [_vp]),
    "kipp_weights_tensor": (_i, [_vp, _i, POINTER(TensorInfo)]),
    "kipp_weights_find": (_i, [_vp, c_char_p, POINTER(TensorInfo)]),
    "kipp_weights_check": (_i, [_vp, c_char_p]),
    "kipp_weights_compare": (_i, [_vp, c_char_p, _cpp]),
    "kipp_engine_open": (_i, [c_char_p, POINTER(EngineOptions), POINTER(_vp)]),
    "kipp_engine_create": (_i, [c_char_p, c_char_p, TENSOR_PROVIDER, _vp, POINTER(ExternalPart), _i,
                                POINTER(EngineOptions), POINTER(_vp)]),
    "kipp_engine_close": (None, [_vp]),
    "kipp_engine_last_error": (c_char_p, [_vp]),
    "kipp_engine_info": (c_char_p, [_vp]),
    "kipp_engine_stream": (_vp, [_vp]),
    "kipp_engine_cache_manager": (_vp, [_vp]),
    "kipp_engine_add_request": (_i, [_vp, c_int64]),
    "kipp_engine_finish": (_i, [_vp, c_int64]),
    "kipp_engine_truncate": (_i, [_vp, c_int64, _i]),
    "kipp_engine_is_live": (_i, [_vp, c_int64]),
    "kipp_engine_length": (_i, [_vp, c_int64]),
    "kipp_engine_step": (_i, [_vp, POINTER(StepEntryC), _i, POINTER(_vp), _ip]),
    "kipp_engine_read_logits": (_i, [_vp, _vp, c_size_t]),
    "kipp_engine_synchronize": (_i, [_vp]),
    "kipp_engine_profile": (_i, [_vp, _i]),
    "kipp_engine_profile_json": (c_char_p, [_vp]),
    "kipp_engine_last_rows": (_i, [_vp]),
    "kipp_engine_debug_set_status": (_i, [_vp, _i, _i]),
    "kipp_engine_decode_burst": (_i, [_vp, POINTER(c_int64), POINTER(c_int32), _i, _i, _vp]),
    "kipp_sample_default_params": (None, [POINTER(SampleParams)]),
    "kipp_engine_sample": (_i, [_vp, POINTER(SampleParams), POINTER(c_uint64), _i, POINTER(c_int32)]),
    "kipp_engine_debug_part": (_i, [_vp, POINTER(StepEntryC), _i, _i, c_char_p, _vp, _vp, _vp]),
    "kipp_scheduler_create": (_i, [_vp, _i, _ip, _ip, _i, _i, POINTER(SchedulerOptions), POINTER(_vp)]),
    "kipp_scheduler_destroy": (None, [_vp]),
    "kipp_scheduler_last_error": (c_char_p, [_vp]),
    "kipp_scheduler_submit": (_i, [_vp, POINTER(GenerationRequest)]),
    "kipp_scheduler_has_work": (_i, [_vp]),
    "kipp_scheduler_schedule": (_i, [_vp, POINTER(PlanEntry), _i, _ip]),
    "kipp_scheduler_tokens": (_i, [_vp, c_int64, _i, _i, POINTER(c_int32)]),
    "kipp_scheduler_complete": (_i, [_vp, POINTER(c_int32), _i]),
    "kipp_scheduler_poll": (_i, [_vp, c_int64, POINTER(GenerationState)]),
    "kipp_scheduler_output": (_i, [_vp, c_int64, POINTER(c_int32), _i, _ip]),
    "kipp_scheduler_abort": (_i, [_vp, c_int64]),
    "kipp_scheduler_forget": (_i, [_vp, c_int64]),
    "kipp_scheduler_list": (_i, [_vp, _i, POINTER(c_int64), _i, _ip]),
    "kipp_scheduler_rng_state": (c_uint64, [_vp, c_int64]),
    "kipp_scheduler_stats": (None, [_vp, _llp]),
    "kipp_engine_scheduler_configure": (_i, [_vp, POINTER(SchedulerOptions)]),
    "kipp_engine_scheduler": (_vp, [_vp]),
    "kipp_engine_run": (_i, [_vp, _i, _ip]),
}

_lib = None


def lib() -> ctypes.CDLL:
    """The host core, built at first use (there is no Python stand-in)."""
    global _lib
    if _lib is None:
        from .csrc import build
        loaded = build.load_host_library()
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(loaded, name)
            fn.restype, fn.argtypes = res, args
        _lib = loaded
    return _lib


def _text(b) -> str:
    return b.decode("utf-8", "replace") if b else ""


def raise_for(code: int, message: str):
    """The exception of a kipp_result."""
    from .cache.pages import OutOfPages
    from .cache.slots import OutOfSlots
    from .config.base import ConfigError
    from .weights.loader import WeightError
    if code in (E_CONFIG, E_UNSUPPORTED):
        raise ConfigError(message)
    if code == E_WEIGHTS:
        raise WeightError.from_message(message)
    if code == E_OUT_OF_PAGES:
        raise OutOfPages(message)
    if code == E_OUT_OF_SLOTS:
        raise OutOfSlots(message)
    if code == E_MEMORY:
        raise MemoryError(message)
    if code == E_ARGUMENT:
        raise ValueError(message)
    if code == E_KERNEL:
        raise KernelError(message)
    if code == E_IO:
        raise OSError(message)
    raise RuntimeError(f"{_text(lib().kipp_result_name(code))}: {message}")


def check(code: int, engine=None, scheduler=None) -> None:
    """Raise for a non-zero result of a library call (the text comes from the
    engine, the scheduler or the thread's last error)."""
    if code == OK:
        return
    L = lib()
    if engine is not None:
        message = _text(L.kipp_engine_last_error(engine))
    elif scheduler is not None:
        message = _text(L.kipp_scheduler_last_error(scheduler))
    else:
        message = _text(L.kipp_last_error())
    raise_for(code, message)


def text_result(fn, *args) -> str:
    """Call ``fn(*args, &text)`` and return the text."""
    out = c_char_p()
    check(fn(*args, ctypes.byref(out)))
    return _text(out.value)


__all__ = ["lib", "check", "raise_for", "text_result", "KernelError", "EngineOptions", "TensorInfo", "TensorView",
           "ExternalCall", "ExternalPart", "EXTERNAL_FORWARD", "TENSOR_PROVIDER", "StepEntryC", "SampleParams",
           "SchedulerOptions", "GenerationRequest", "GenerationState", "PlanEntry", "c_double"]
